"""CPU-side checks: the product library loads and exports the whole ABI, refuses to run
without a GPU, and the host-side rules of the oracle (shapes, padding, rounding)."""
import ctypes as C
import os
import re

import numpy as np

import oracle_paths
import pyb2vx as B

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "b2vx.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b2vx_[a-z0-9_]+)\s*\(", text)))


def test_product_library_exports_every_declared_symbol():
    assert os.path.exists(B.PRODUCT_LIB), "build first: python -c 'import __graft_entry__ as g; g.build()'"
    lib = C.CDLL(B.PRODUCT_LIB)
    names = declared_symbols()
    assert len(names) >= 25
    for n in names:
        assert hasattr(lib, n), n


def test_oracle_library_exports_the_same_abi(oracle_lib):
    """The oracle serves the graph ABI; the allocation-free convolution and the tensor-pipe measurement are
    CUDA-only additions."""
    for n in declared_symbols():
        if n.endswith("_noalloc") or n == "b2vx_measure_int8_peak":
            continue
        assert hasattr(oracle_lib, n), n


def test_product_has_no_cpu_fallback():
    """Without a CUDA device graph creation fails with a clear message."""
    lib = B.load(B.PRODUCT_LIB)
    if lib.b2vx_device_count() > 0:
        return
    try:
        B.Graph(lib)
    except B.B2vxError as e:
        assert e.status == 6 and "no CUDA device" in str(e)
    else:
        raise AssertionError("graph creation succeeded without a GPU")


def _ops():
    lib = C.CDLL(oracle_paths.ORACLE_OPS_LIB)
    lib.orc_rint.restype = C.c_double
    lib.orc_rint.argtypes = [C.c_double]
    lib.orc_fp32_to_affine.restype = C.c_int32
    lib.orc_fp32_to_affine.argtypes = [C.c_float, C.c_float, C.c_int32, C.c_int32]
    lib.orc_filter_size.restype = C.c_uint32
    lib.orc_filter_size.argtypes = [C.c_uint32] * 6 + [C.c_int32]
    lib.orc_same_valid_padding.argtypes = [C.c_uint32] * 4 + [C.c_int32, C.POINTER(C.c_uint32)]
    return lib


def test_rounding_rule(oracle_lib):
    ops = _ops()
    # ties to even, everything else to nearest (vsi_rint)
    for x, want in [(0.5, 0), (1.5, 2), (2.5, 2), (3.5, 4), (-0.5, 0), (-1.5, -2), (-2.5, -2), (2.4999, 2), (2.5001, 3),
                    (-7.5, -8), (1e6 + 0.5, 1e6)]:
        assert ops.orc_rint(x) == want, x
    # the float-add quirk of floorf(fabsf(x)+0.5f): the largest float below 0.5 rounds up
    assert ops.orc_rint(float(np.nextafter(np.float32(0.5), np.float32(0)))) == 1
    # saturation and infinities
    assert ops.orc_fp32_to_affine(1e9, 0.5, 3, B.DT_UINT8) == 255
    assert ops.orc_fp32_to_affine(-1e9, 0.5, 3, B.DT_UINT8) == 0
    assert ops.orc_fp32_to_affine(float("inf"), 0.5, 3, B.DT_INT8) == 127
    assert ops.orc_fp32_to_affine(float("-inf"), 0.5, 3, B.DT_INT8) == -128
    assert ops.orc_fp32_to_affine(1.25, 0.5, 10, B.DT_UINT8) == 12   # 2.5 -> 2, +10


def test_shape_rules():
    ops = _ops()
    pad = (C.c_uint32 * 2)()
    # SAME 3x3 stride 1 on 56 -> 1/1; stride 2 on 56 -> out 28, total 1 -> front 0, end 1
    ops.orc_same_valid_padding(56, 3, 1, 1, B.PAD_SAME, pad); assert list(pad) == [1, 1]
    ops.orc_same_valid_padding(56, 3, 2, 1, B.PAD_SAME, pad); assert list(pad) == [0, 1]
    ops.orc_same_valid_padding(224, 7, 2, 1, B.PAD_SAME, pad); assert list(pad) == [2, 3]
    ops.orc_same_valid_padding(28, 5, 1, 1, B.PAD_VALID, pad); assert list(pad) == [0, 0]
    assert ops.orc_filter_size(56, 3, 1, 1, 1, 1, B.ROUND_FLOOR) == 56
    assert ops.orc_filter_size(56, 3, 0, 1, 2, 1, B.ROUND_FLOOR) == 28
    assert ops.orc_filter_size(112, 3, 0, 1, 2, 1, B.ROUND_CEILING) == 56
    assert ops.orc_filter_size(112, 3, 0, 0, 2, 1, B.ROUND_FLOOR) == 55
    assert ops.orc_filter_size(9, 3, 0, 0, 1, 3, B.ROUND_FLOOR) == 3   # dilation 3 -> effective 7
    assert ops.orc_filter_size(9, 3, 0, 0, 1, 0, B.ROUND_FLOOR) == 7   # dilation 0 means 1


def test_oracle_graph_shape_inference(oracle_lib):
    g = B.Graph(oracle_lib)
    x = g.tensor(B.DT_UINT8, [224, 224, 3, 2], B.ATTR_INPUT, scale=0.02, zero_point=128)
    w = g.tensor(B.DT_INT8, [7, 7, 3, 64], B.ATTR_CONSTANT, scales=[0.01] * 64, channel_dim=3,
                 data=np.zeros((64, 3, 7, 7), np.int8))
    y = g.tensor(B.DT_UINT8, [], B.ATTR_TRANSIENT, scale=0.1, zero_point=0)
    p = g.tensor(B.DT_UINT8, [], B.ATTR_OUTPUT, scale=0.1, zero_point=0)
    g.conv2d(x, w, None, y, stride=(2, 2), pad=(3, 3, 3, 3))
    g.pool2d(y, p, B.POOL_MAX, (3, 3), (2, 2), pad=(0, 1, 0, 1), round_type=B.ROUND_CEILING)
    g.compile()
    assert g.shape(y) == [112, 112, 64, 2]
    assert g.shape(p) == [56, 56, 64, 2]
    g.close()


def test_oracle_rejects_mismatched_shapes(oracle_lib):
    g = B.Graph(oracle_lib)
    a = g.tensor(B.DT_UINT8, [4, 4, 8, 1], B.ATTR_INPUT, scale=0.1, zero_point=0)
    b = g.tensor(B.DT_UINT8, [4, 3, 8, 1], B.ATTR_INPUT, scale=0.1, zero_point=0)
    y = g.tensor(B.DT_UINT8, [], B.ATTR_OUTPUT, scale=0.1, zero_point=0)
    g.add(a, b, y)
    try:
        g.compile()
    except B.B2vxError as e:
        assert e.status == 3
    else:
        raise AssertionError("shape mismatch accepted")
    g.close()


def test_oracle_l2_pool_is_root_mean_square_of_the_valid_taps(oracle_lib):
    """Pool2d L2 as this repository defines it (the reference lowers the type but states no formula): the oracle against
    a float64 numpy restatement, within one quantization step."""
    import graph_cases as G
    W = H = 10
    C, N, k, stride, pad = 16, 2, 3, 2, 1
    in_q, out_q = (0.05, 120), (0.03, 0)
    out, _ = G.run_case(oracle_lib, G.pool_q(W, H, C, N, B.POOL_L2, (k, k), (stride, stride), pad=(pad, pad, pad, pad), in_q=in_q, out_q=out_q), seed=9)
    rng = np.random.default_rng(9)
    x = G._act(rng, [W, H, C, N]).astype(np.float64)
    real = (x - in_q[1]) * in_q[0]
    Ho = (H + 2 * pad - k) // stride + 1
    want = np.zeros((N, C, Ho, Ho))
    for ho in range(Ho):
        for wo in range(Ho):
            h0, w0 = ho * stride - pad, wo * stride - pad
            patch = real[:, :, max(h0, 0):min(h0 + k, H), max(w0, 0):min(w0 + k, W)]
            want[:, :, ho, wo] = np.sqrt((patch ** 2).mean(axis=(2, 3)))
    q = np.clip(np.rint(want / out_q[0]) + out_q[1], 0, 255)
    assert np.abs(out[0].astype(np.float64) - q).max() <= 1
