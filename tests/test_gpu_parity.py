"""GPU parity: the CUDA library against the reference's vectors and the CPU oracle.

All calls go through the C ABI (pyb2vx).  Integer outputs must be bit-exact;
float32 softmax is compared within 1e-5 (device expf vs libm expf); float32
convolution/pooling/FC replay the oracle's operation order without fused
multiply-add and must be bit-exact too.
"""
import os

import numpy as np
import pytest

import graph_cases as G
import oracle_paths
import pyb2vx as B

pytestmark = pytest.mark.gpu

SOFTMAX_TOL = 1e-5


@pytest.fixture(params=["tensorcore", "cudacore"])
def conv_kernel(request):
    """Run a test once with the tensor-core GEMM path and once with the CUDA-core path."""
    old = os.environ.get("B2VX_CONV_KERNEL")
    os.environ["B2VX_CONV_KERNEL"] = "tc" if request.param == "tensorcore" else "simt"
    yield request.param
    if old is None:
        os.environ.pop("B2VX_CONV_KERNEL", None)
    else:
        os.environ["B2VX_CONV_KERNEL"] = old


def test_device_present(product_lib):
    assert product_lib.b2vx_device_count() >= 1


def test_reference_vectors(product_lib, reference_cases, conv_kernel):
    """Every graph of the reference's unit tests: GPU vs the test's own expected vector,
    and GPU vs the oracle output recorded in the fixture (bit for bit for integers)."""
    failures = []
    for case in reference_cases:
        g, inputs, expects, recorded = oracle_paths.graph_from_case(product_lib, case)
        try:
            g.compile()
            for tid, arr in inputs:
                g.write(tid, arr)
            g.run()
            is_softmax = any(n["kind"] == B.NODE_SOFTMAX for n in case["nodes"])
            for tid, want, tol in expects:
                got = g.read(tid).reshape(-1)
                if want.dtype == np.float32:
                    if not np.allclose(got, want, rtol=0, atol=max(tol, 1e-5)):
                        failures.append("%s: float mismatch vs reference vector %g" % (case["name"], np.abs(got - want).max()))
                else:
                    d = np.abs(got.astype(np.int64) - want.astype(np.int64)).max()
                    if d > tol:
                        failures.append("%s: |gpu - reference vector| = %d > %g" % (case["name"], d, tol))
            for tid, want in recorded.items():
                got = g.read(tid).reshape(-1)
                if is_softmax:
                    ok = np.allclose(got, want, rtol=0, atol=SOFTMAX_TOL)
                else:
                    ok = np.array_equal(got.view(np.uint8), want.view(np.uint8))
                if not ok:
                    failures.append("%s: gpu differs from oracle output" % case["name"])
        except B.B2vxError as e:
            failures.append("%s: %s" % (case["name"], e))
        finally:
            g.close()
    assert not failures, "\n".join(failures[:40])


CONV_CASES = {
    # the single-conv sweep of the benchmark configuration at small batch, plus its 1x1 and stride-2 variants
    "cfg2_3x3_n1": G.conv2d_q(56, 56, 64, 1, 3, 3, 64, relu=True),
    "cfg2_3x3_n3": G.conv2d_q(56, 56, 64, 3, 3, 3, 64, relu=True),
    "cfg2_1x1": G.conv2d_q(56, 56, 64, 2, 1, 1, 64, relu=True),
    # more than eight 128-row tiles per SM with a short K: tiles of 65-128 columns also go one per warp group
    "many_tiles_16_96_u8": G.conv2d_q(448, 400, 16, 1, 1, 1, 96, w_kind="u8", relu=True),
    "many_tiles_64_128": G.conv2d_q(224, 224, 64, 4, 1, 1, 128, in_q=(0.02, 3)),
    "cfg2_3x3_s2": G.conv2d_q(56, 56, 64, 2, 3, 3, 64, stride=(2, 2), relu=True),
    # channel counts that need padding, odd sizes, ragged tiles
    "c24_oc40": G.conv2d_q(13, 11, 24, 2, 3, 3, 40),
    "c3_stem7x7": G.conv2d_q(32, 32, 3, 2, 7, 7, 64, stride=(2, 2), pad_type=B.PAD_AUTO, pad=(3, 3, 3, 3)),
    # first layers (graph inputs with few channels) at strides 2 and 4: channel counts 1-8, filter rows of 2-8 taps, odd and
    # even left padding, a weight zero point (ones row), signed input
    "stem_3x3_s2_c3_u8": G.conv2d_q(224, 224, 3, 2, 3, 3, 32, stride=(2, 2), w_kind="u8", relu=True),
    "stem_7x7_s2_c3": G.conv2d_q(75, 61, 3, 3, 7, 7, 64, stride=(2, 2), pad_type=B.PAD_AUTO, pad=(3, 3, 3, 3), relu=True),
    "stem_5x5_s2_c1": G.conv2d_q(28, 28, 1, 2, 5, 5, 20, stride=(2, 2), in_q=(0.02, 7)),
    "stem_8x3_s2_c8_nopad": G.conv2d_q(40, 21, 8, 2, 8, 3, 24, stride=(2, 2), pad_type=B.PAD_VALID),
    "stem_2x2_s2_c4_s8in": G.conv2d_q(30, 30, 4, 2, 2, 2, 16, stride=(2, 2), pad_type=B.PAD_VALID, x_dtype=B.DT_INT8, in_q=(0.02, -5)),
    "stem_6x6_s2_pad2": G.conv2d_q(33, 35, 2, 1, 6, 6, 48, stride=(2, 2), pad_type=B.PAD_AUTO, pad=(2, 2, 2, 2), w_kind="u8"),
    "stem_4x4_s4_c3": G.conv2d_q(64, 48, 3, 2, 4, 4, 96, stride=(4, 4), pad_type=B.PAD_VALID),
    "stem_7x1_s2": G.conv2d_q(50, 9, 3, 1, 7, 1, 16, stride=(2, 2), pad_type=B.PAD_AUTO, pad=(3, 3, 0, 0)),
    "c1_5x5_valid": G.conv2d_q(28, 28, 1, 2, 5, 5, 20, pad_type=B.PAD_VALID, w_kind="u8z128", in_q=(1 / 255.0, 0), out_q=(0.05, 128)),
    "u8_weights_zp": G.conv2d_q(10, 9, 20, 2, 3, 3, 50, w_kind="u8", out_q=(0.3, 121)),
    "u8_weights_1x1": G.conv2d_q(7, 7, 96, 3, 1, 1, 24, w_kind="u8", out_q=(0.2, 130)),
    "s8_act_s8_w": G.conv2d_q(9, 9, 16, 1, 3, 3, 32, x_dtype=B.DT_INT8, w_kind="s8", in_q=(0.5, -1), out_q=(1.5, -3), out_dtype=B.DT_INT8),
    "dilated": G.conv2d_q(17, 15, 32, 1, 3, 3, 32, dilation=(2, 2)),
    "oc_320_two_n_tiles": G.conv2d_q(7, 7, 64, 4, 1, 1, 320),
    "oc_1024_k_2048": G.conv2d_q(4, 4, 2048, 2, 1, 1, 1024, in_q=(0.02, 128), out_q=(0.6, 0)),
    "explicit_pad_asym": G.conv2d_q(12, 12, 16, 1, 3, 3, 16, stride=(2, 2), pad_type=B.PAD_AUTO, pad=(0, 1, 0, 1)),
    "no_bias": G.conv2d_q(8, 8, 16, 1, 3, 3, 16, bias=False),
    "single_pixel": G.conv2d_q(1, 1, 64, 1, 1, 1, 16),
    # non-zero input zero point with padding: border classes in the tensor-core epilogue
    "zp_pad_5x5_s2": G.conv2d_q(23, 19, 32, 2, 5, 5, 48, stride=(2, 2)),
    "zp_pad_dil3": G.conv2d_q(20, 20, 16, 1, 3, 3, 16, dilation=(3, 3)),
    "zp_pad_window_wider_than_input": G.conv2d_q(3, 2, 16, 2, 5, 5, 16),
    # uint8 weights with a zero point other than 128: the ones row / S column, alone and with borders,
    # over several N tiles
    "u8_w_oc300": G.conv2d_q(9, 9, 32, 2, 1, 1, 300, w_kind="u8"),
    "u8_w_3x3_oc272_pad": G.conv2d_q(12, 10, 48, 1, 3, 3, 272, w_kind="u8"),
    "u8_w_stem": G.conv2d_q(30, 30, 3, 2, 3, 3, 32, stride=(2, 2), w_kind="u8", in_q=(0.02, 114)),
    # wide first-layer filters: the row-of-8 im2col, with and without a weight zero point
    "stem5x5_c3_u8w": G.conv2d_q(31, 29, 3, 2, 5, 5, 24, w_kind="u8", in_q=(0.02, 114)),
    "stem8x6_c4_s1": G.conv2d_q(20, 17, 4, 1, 8, 6, 16, in_q=(0.03, 9)),
    # weight tile resident in shared memory with several channel blocks per tap; narrow tiles on epilogue teams,
    # with more tiles than accumulator buffers per CTA
    "resident_c96_3x3_oc32": G.conv2d_q(33, 29, 96, 3, 3, 3, 32),
    "resident_c160_5x5_oc16_u8w": G.conv2d_q(21, 17, 160, 2, 5, 5, 16, w_kind="u8"),
    "teams_many_tiles_oc48": G.conv2d_q(120, 110, 16, 2, 3, 3, 48, relu=True),
    # halo mode of the implicit convolution (stride 1, resident weights, 64-byte channel blocks): three channel blocks per
    # patch; a 5x5 window with a weight zero point on an output whose right and bottom tiles are ragged; signed bytes
    "halo_c192_3x3_oc32": G.conv2d_q(24, 32, 192, 2, 3, 3, 32),
    "halo_c64_5x5_oc16_u8w_ragged": G.conv2d_q(63, 47, 64, 2, 5, 5, 16, w_kind="u8"),
    "halo_c64_3x3_s8": G.conv2d_q(40, 48, 64, 1, 3, 3, 64, x_dtype=B.DT_INT8, w_kind="s8", in_q=(0.5, -1), out_q=(1.5, -3), out_dtype=B.DT_INT8),
}

HALO_CASES = ["cfg2_3x3_n1", "cfg2_3x3_n3", "halo_c192_3x3_oc32", "halo_c64_5x5_oc16_u8w_ragged", "halo_c64_3x3_s8"]


@pytest.mark.parametrize("name", sorted(CONV_CASES))
def test_conv2d_matches_oracle(oracle_lib, product_lib, conv_kernel, name):
    want, _ = G.run_case(oracle_lib, CONV_CASES[name], seed=11)
    got, kernels = G.run_case(product_lib, CONV_CASES[name], seed=11)
    G.assert_same(want, got)
    names = [k["name"] for k in kernels]
    if conv_kernel == "cudacore":
        assert not any(n.startswith("gemm_i8_tc") for n in names)


@pytest.mark.parametrize("name", HALO_CASES)
def test_halo_mode_is_taken(product_lib, name):
    if os.environ.get("B2VX_TC_HALO") == "0":
        pytest.skip("halo mode switched off by the environment")
    os.environ.pop("B2VX_CONV_KERNEL", None)
    _, kernels = G.run_case(product_lib, CONV_CASES[name], seed=11)
    assert any(k["name"].startswith("gemm_i8_tc(halo") for k in kernels), [k["name"] for k in kernels]


def test_padded_conv_with_zero_point_is_implicit(product_lib):
    """The benchmark's 3x3 SAME convolution (input zero point 128) runs as an implicit GEMM: no im2col pass."""
    os.environ.pop("B2VX_CONV_KERNEL", None)
    _, kernels = G.run_case(product_lib, CONV_CASES["cfg2_3x3_n3"], seed=1)
    names = [k["name"] for k in kernels]
    assert ("gemm_i8_tc(halo)" in names or "gemm_i8_tc(implicit)" in names) and not any(n.startswith("im2col") for n in names), names


def test_uint8_weight_zero_point_runs_on_tensor_cores(product_lib):
    os.environ.pop("B2VX_CONV_KERNEL", None)
    _, kernels = G.run_case(product_lib, CONV_CASES["u8_weights_1x1"], seed=1)
    assert any(k["name"].startswith("gemm_i8_tc") for k in kernels), [k["name"] for k in kernels]


def test_tensor_core_path_is_taken(product_lib):
    """With the default setting a plain int8 convolution runs on the tcgen05 GEMM."""
    os.environ.pop("B2VX_CONV_KERNEL", None)
    _, kernels = G.run_case(product_lib, CONV_CASES["cfg2_1x1"], seed=1)
    assert any(k["name"].startswith("gemm_i8_tc") for k in kernels), [k["name"] for k in kernels]


DEPTHWISE_CASES = {
    "dw3x3_s1": G.depthwise_q(28, 28, 32, 2, 3, 3),
    "dw3x3_s2": G.depthwise_q(28, 28, 96, 2, 3, 3, stride=(2, 2)),
    "dw_c24": G.depthwise_q(15, 15, 24, 1, 3, 3),
    "dw_mult2": G.depthwise_q(9, 9, 6, 2, 3, 3, multiplier=2),
    "dw_s8pc": G.depthwise_q(14, 14, 64, 2, 3, 3, w_kind="s8pc"),
    "dw5x5": G.depthwise_q(11, 13, 16, 1, 5, 5, relu6=False),
    # strip form (3x3, stride 1 or 2): whole images per tile with an odd batch, ragged widths and channel counts,
    # one 16-channel chunk, VALID and explicit one-sided padding, signed input bytes, wide rows
    "dw_7x7_c960_n3": G.depthwise_q(7, 7, 960, 3, 3, 3),
    "dw_7x7_c16_n9": G.depthwise_q(7, 7, 16, 9, 3, 3),
    "dw_14x14_c384_s2_n3": G.depthwise_q(14, 14, 384, 3, 3, 3, stride=(2, 2)),
    "dw_13x9_c144": G.depthwise_q(13, 9, 144, 2, 3, 3),
    "dw_56x56_c144_s2": G.depthwise_q(56, 56, 144, 1, 3, 3, stride=(2, 2)),
    "dw_112x112_c32": G.depthwise_q(112, 112, 32, 1, 3, 3),
    "dw_valid_s1": G.depthwise_q(19, 11, 40, 2, 3, 3, pad_type=B.PAD_VALID),
    "dw_valid_s2": G.depthwise_q(19, 12, 40, 2, 3, 3, stride=(2, 2), pad_type=B.PAD_VALID),
    "dw_pad_1002": G.depthwise_q(21, 10, 48, 2, 3, 3, pad_type=B.PAD_AUTO, pad=(1, 0, 0, 2)),
    "dw_s8_input": G.depthwise_q(17, 17, 72, 2, 3, 3, x_dtype=B.DT_INT8, in_q=(0.03, -8), w_kind="s8pc"),
    "dw_s8_input_s2": G.depthwise_q(17, 18, 24, 2, 3, 3, stride=(2, 2), x_dtype=B.DT_INT8, in_q=(0.03, 5)),
    "dw_1x1_image": G.depthwise_q(1, 1, 64, 5, 3, 3),
    "dw_3x40_c8": G.depthwise_q(40, 3, 8, 1, 3, 3),
}


@pytest.mark.parametrize("name", sorted(DEPTHWISE_CASES))
def test_depthwise_matches_oracle(oracle_lib, product_lib, name):
    want, _ = G.run_case(oracle_lib, DEPTHWISE_CASES[name], seed=5)
    got, _ = G.run_case(product_lib, DEPTHWISE_CASES[name], seed=5)
    G.assert_same(want, got)


def test_strip_form_equals_sixteen_channel_form(product_lib):
    """B2VX_DW_STRIP=0 selects the kernel that owns sixteen channels of two pixels per thread: same bytes."""
    for name in ("dw3x3_s1", "dw3x3_s2", "dw_13x9_c144", "dw_7x7_c960_n3"):
        got, kernels = G.run_case(product_lib, DEPTHWISE_CASES[name], seed=5)
        assert any(k["name"] == "depthwise_q16" for k in kernels), [k["name"] for k in kernels]
        os.environ["B2VX_DW_STRIP"] = "0"
        try:
            other, _ = G.run_case(product_lib, DEPTHWISE_CASES[name], seed=5)
        finally:
            os.environ.pop("B2VX_DW_STRIP", None)
        G.assert_same(got, other)


@pytest.mark.parametrize("name", sorted(n for n in DEPTHWISE_CASES if n not in ("dw_mult2", "dw5x5")))
def test_pipelined_depthwise_matches_oracle(oracle_lib, product_lib, name):
    """B2VX_DW_PIPE=1 sends every 3x3 stride-1/2 layer through the persistent, double-buffered form that large
    layers take by default (a block walks over several tiles of its channel slab)."""
    want, _ = G.run_case(oracle_lib, DEPTHWISE_CASES[name], seed=6)
    os.environ["B2VX_DW_PIPE"] = "1"
    try:
        got, _ = G.run_case(product_lib, DEPTHWISE_CASES[name], seed=6)
    finally:
        os.environ.pop("B2VX_DW_PIPE", None)
    G.assert_same(want, got)


def test_pipelined_depthwise_many_tiles_per_block(oracle_lib, product_lib):
    """Enough tiles that every persistent block takes several (both buffers in use, last round ragged).  The first
    case is large enough to take the pipelined form by itself; the others are sent there."""
    cases = [(G.depthwise_q(56, 56, 32, 120, 3, 3), None),
             (G.depthwise_q(57, 55, 16, 500, 3, 3, stride=(2, 2)), "1"),
             (G.depthwise_q(28, 28, 24, 200, 3, 3, x_dtype=B.DT_INT8, in_q=(0.03, 3)), "1")]
    for case, pipe in cases:
        want, _ = G.run_case(oracle_lib, case, seed=8)
        for env in (pipe, "0"):
            if env is not None:
                os.environ["B2VX_DW_PIPE"] = env
            try:
                got, _ = G.run_case(product_lib, case, seed=8)
            finally:
                os.environ.pop("B2VX_DW_PIPE", None)
            G.assert_same(want, got)


FC_CASES = {
    "fc_1024_m16": G.fc_q(1024, 1024, 16),
    "fc_1024_m1": G.fc_q(1024, 1024, 1),
    "fc_1024_m130": G.fc_q(1024, 1024, 130),
    "fc_k500_n10": G.fc_q(500, 10, 5, w_kind="u8z128"),
    "fc_k800_from4d": G.fc_q(800, 500, 3, from_4d=(4, 4, 50), w_kind="u8z128"),
    "fc_u8_zp": G.fc_q(1280, 1000, 2, w_kind="u8"),
    "fc_2048_1000": G.fc_q(2048, 1000, 4),
    # the row-count variants of the small-M kernel, ragged channel counts, a weight zero point
    "fc_m7_n1001": G.fc_q(768, 1001, 7),
    "fc_m8_n30": G.fc_q(4096, 30, 8),
    "fc_m16_n30": G.fc_q(4096, 30, 16),
    "fc_m3_u8zp": G.fc_q(512, 200, 3, w_kind="u8"),
    "fc_m9_u8zp": G.fc_q(1024, 64, 9, w_kind="u8"),
    "fc_m6_u8zp": G.fc_q(1024, 64, 6, w_kind="u8"),
    # resident weight tile on the plain GEMM path, many row tiles
    "fc_k512_n64_m3000": G.fc_q(512, 64, 3000),
    "fc_k320_n48_m700_u8zp": G.fc_q(320, 48, 700, w_kind="u8"),
}


@pytest.mark.parametrize("name", sorted(FC_CASES))
def test_fully_connected_matches_oracle(oracle_lib, product_lib, conv_kernel, name):
    want, _ = G.run_case(oracle_lib, FC_CASES[name], seed=3)
    got, _ = G.run_case(product_lib, FC_CASES[name], seed=3)
    G.assert_same(want, got)


@pytest.mark.parametrize("name", ["fc_m8_n30", "fc_1024_m1", "fc_u8_zp", "fc_k800_from4d"])
def test_small_m_fc_on_tensor_cores_matches_oracle(oracle_lib, product_lib, name):
    """The same few-row shapes kept on the tcgen05 kernel (128-row tiles, mostly out of bounds)."""
    want, _ = G.run_case(oracle_lib, FC_CASES[name], seed=3)
    os.environ["B2VX_FC_SMALL_M"] = "0"
    os.environ.pop("B2VX_CONV_KERNEL", None)
    try:
        got, kernels = G.run_case(product_lib, FC_CASES[name], seed=3)
    finally:
        os.environ.pop("B2VX_FC_SMALL_M", None)
    assert any(k["name"].startswith("gemm_i8_tc") for k in kernels), [k["name"] for k in kernels]
    G.assert_same(want, got)


SMALL_M = ["fc_1024_m1", "fc_1024_m16", "fc_2048_1000", "fc_k500_n10", "fc_k800_from4d", "fc_m16_n30", "fc_m3_u8zp",
           "fc_m6_u8zp", "fc_m7_n1001", "fc_m8_n30", "fc_m9_u8zp", "fc_u8_zp"]


@pytest.mark.parametrize("name", SMALL_M)
@pytest.mark.parametrize("fc_mma", ["0", "1"])
def test_small_m_fc_both_kernels_match_oracle(oracle_lib, product_lib, name, fc_mma):
    """Every few-row shape on the dp4a kernel (B2VX_FC_MMA=0; up to 16 rows) and on the mma.sync kernel (=1): ragged
    channel counts, K that is not a multiple of 64, a weight zero point, one to sixteen rows."""
    want, _ = G.run_case(oracle_lib, FC_CASES[name], seed=3)
    os.environ["B2VX_FC_MMA"] = fc_mma
    os.environ.pop("B2VX_CONV_KERNEL", None)
    try:
        got, kernels = G.run_case(product_lib, FC_CASES[name], seed=3)
    finally:
        os.environ.pop("B2VX_FC_MMA", None)
    assert any(k["name"] == "fc_small_m" for k in kernels), [k["name"] for k in kernels]
    G.assert_same(want, got)


def test_small_m_fc_kernel_is_taken(product_lib):
    _, kernels = G.run_case(product_lib, FC_CASES["fc_1024_m1"], seed=3)
    assert [k["name"] for k in kernels if k["name"].startswith(("fc_", "gemm_"))] == ["fc_small_m"], [k["name"] for k in kernels]


POOL_CASES = {
    "max2x2": G.pool_q(24, 24, 20, 2, B.POOL_MAX, (2, 2), (2, 2)),
    "max3x3s2_ceil": G.pool_q(112, 112, 64, 1, B.POOL_MAX, (3, 3), (2, 2), pad=(0, 1, 0, 1), round_type=B.ROUND_CEILING),
    "max_requant": G.pool_q(9, 9, 16, 1, B.POOL_MAX, (3, 3), (1, 1), pad=(1, 1, 1, 1), out_q=(0.07, 10)),
    # the 2 x 2-outputs-per-thread kernel: padding on every side, odd output extents (a thread's second row / column missing),
    # signed bytes, a 2x2 window on odd inputs, ceiling mode with windows hanging over the right and bottom edges
    "max3x3s2_pad1": G.pool_q(28, 28, 48, 2, B.POOL_MAX, (3, 3), (2, 2), pad=(1, 1, 1, 1)),
    "max3x3s2_odd": G.pool_q(15, 13, 32, 3, B.POOL_MAX, (3, 3), (2, 2), pad=(1, 0, 0, 1)),
    "max3x3s2_s8": G.pool_q(11, 9, 16, 2, B.POOL_MAX, (3, 3), (2, 2), pad=(2, 2, 2, 2), in_q=(0.1, -5), dtype=B.DT_INT8),
    "max2x2s2_odd_ceil": G.pool_q(9, 7, 32, 2, B.POOL_MAX, (2, 2), (2, 2), round_type=B.ROUND_CEILING),
    "max3x3s2_tiny": G.pool_q(3, 3, 16, 1, B.POOL_MAX, (3, 3), (2, 2), pad=(1, 1, 1, 1)),
    "avg7x7_global": G.pool_q(7, 7, 2048, 2, B.POOL_AVG, (7, 7), (7, 7), out_q=(0.04, 7)),
    "avg_pad": G.pool_q(10, 10, 32, 1, B.POOL_AVG, (3, 3), (2, 2), pad=(1, 1, 1, 1)),
    "avg_android_pad": G.pool_q(10, 10, 32, 1, B.POOL_AVG_ANDROID, (3, 3), (2, 2), pad=(1, 1, 1, 1)),
    "avg_s8": G.pool_q(8, 8, 16, 1, B.POOL_AVG, (2, 2), (2, 2), in_q=(0.1, -5), dtype=B.DT_INT8),
    # L2: sqrt of the mean square over the taps inside the input (parity unpinned: the reference holds no vector)
    "l2_3x3_pad": G.pool_q(10, 10, 32, 2, B.POOL_L2, (3, 3), (2, 2), pad=(1, 1, 1, 1), in_q=(0.05, 120), out_q=(0.03, 0)),
    "l2_global_s8": G.pool_q(7, 7, 48, 2, B.POOL_L2, (7, 7), (7, 7), in_q=(0.1, -5), out_q=(0.08, -128), dtype=B.DT_INT8),
}


@pytest.mark.parametrize("name", sorted(POOL_CASES))
def test_pool_matches_oracle(oracle_lib, product_lib, name):
    want, _ = G.run_case(oracle_lib, POOL_CASES[name], seed=9)
    got, _ = G.run_case(product_lib, POOL_CASES[name], seed=9)
    G.assert_same(want, got)


ELTWISE_CASES = {
    "add_resnet": G.add_q([56, 56, 256, 1], relu=True),
    "add_c24": G.add_q([14, 14, 24, 2]),
    "add_1m": G.add_q([1 << 20]),
    "relu": G.relu_q([14, 14, 40, 2]),
    "relu6": G.relu_q([14, 14, 40, 2], six=True, qi=(0.05, 100), qo=(0.0235, 0)),
}


@pytest.mark.parametrize("name", sorted(ELTWISE_CASES))
def test_elementwise_matches_oracle(oracle_lib, product_lib, name):
    want, _ = G.run_case(oracle_lib, ELTWISE_CASES[name], seed=21)
    got, _ = G.run_case(product_lib, ELTWISE_CASES[name], seed=21)
    G.assert_same(want, got)


def _addn_case(n_in, dims, dtype=B.DT_UINT8):
    def build(g, rng):
        ins = []
        for k in range(n_in):
            if dtype == B.DT_FLOAT32:
                t = g.tensor(dtype, dims, B.ATTR_INPUT)
                a = rng.normal(size=dims[::-1]).astype(np.float32)
            else:
                t = g.tensor(dtype, dims, B.ATTR_INPUT, scale=0.01 + 0.007 * k, zero_point=100 + 9 * k if dtype == B.DT_UINT8 else -3 + k)
                a = rng.integers(0, 256, size=dims[::-1]).astype(np.uint8).view(np.int8 if dtype == B.DT_INT8 else np.uint8)
            ins.append((t, a))
        y = g.tensor(dtype, [], B.ATTR_OUTPUT, **({} if dtype == B.DT_FLOAT32 else dict(scale=0.05, zero_point=120 if dtype == B.DT_UINT8 else 5)))
        g.addn([t for t, _ in ins], y)
        return ins, [y]
    return build


@pytest.mark.parametrize("n_in,dims,dtype", [(2, [14, 14, 24, 2], B.DT_UINT8), (3, [14, 14, 24, 2], B.DT_UINT8), (5, [7, 5, 40, 3], B.DT_INT8),
                                             (16, [33], B.DT_UINT8), (4, [9, 3, 5], B.DT_FLOAT32)])
def test_addn_matches_oracle(oracle_lib, product_lib, n_in, dims, dtype):
    """ops::AddN: two inputs run the Add kernels, more the n-input kernel (the sum stays float32 until the end)."""
    want, _ = G.run_case(oracle_lib, _addn_case(n_in, dims, dtype), seed=5)
    got, kernels = G.run_case(product_lib, _addn_case(n_in, dims, dtype), seed=5)
    assert any(k["name"] == ("addn" if n_in > 2 else ("add_q" if dtype != B.DT_FLOAT32 else "add_f32")) for k in kernels), [k["name"] for k in kernels]
    G.assert_same(want, got)


ADD_QUANTS = {
    # 0.4*i + 0.7*j: one sum in ten lands on a .5 fraction (the arithmetic kernel's exact path)
    "many_ties": dict(qa=(0.02, 128), qb=(0.035, 117), qo=(0.05, 120)),
    "irregular": dict(qa=(0.0213, 7), qb=(0.0347, 250), qo=(0.0512, 33)),
    "coarse_out": dict(qa=(0.11, 100), qb=(0.003, 140), qo=(0.9, 128)),
    "fine_out": dict(qa=(0.05, 120), qb=(0.07, 130), qo=(0.004, 128)),   # saturates most sums
    "extreme": dict(qa=(900.0, 128), qb=(0.5, 3), qo=(0.0001, 10)),      # beyond the fast rounding's range
}


@pytest.mark.parametrize("kernel", ["lut", "alu"])
@pytest.mark.parametrize("quant", sorted(ADD_QUANTS))
def test_add_kernels_match_oracle(oracle_lib, product_lib, kernel, quant):
    """Both quantized-Add kernels (table in shared memory; packed float arithmetic) on every pair of
    input bytes, several times over so that all lanes and both loop iterations are exercised."""
    def build(g, rng):
        n = 65536 * 4
        q = ADD_QUANTS[quant]
        a = g.tensor(B.DT_UINT8, [n], B.ATTR_INPUT, scale=q["qa"][0], zero_point=q["qa"][1])
        b = g.tensor(B.DT_UINT8, [n], B.ATTR_INPUT, scale=q["qb"][0], zero_point=q["qb"][1])
        y = g.tensor(B.DT_UINT8, [], B.ATTR_OUTPUT, scale=q["qo"][0], zero_point=q["qo"][1])
        g.add(a, b, y)
        i = (np.arange(n) * 40503) % 65536           # every (a, b) pair, scattered over lanes
        return [(a, (i >> 8).astype(np.uint8)), (b, (i & 255).astype(np.uint8))], [y]
    want, _ = G.run_case(oracle_lib, build, seed=1)
    os.environ["B2VX_ADD_KERNEL"] = kernel
    try:
        got, kernels = G.run_case(product_lib, build, seed=1)
    finally:
        os.environ.pop("B2VX_ADD_KERNEL", None)
    assert [k["name"] for k in kernels] == ["add_q_lut" if kernel == "lut" else "add_q"]
    G.assert_same(want, got)


BROADCAST_SHAPES = {
    "per_channel": ([8, 6, 20, 2], [1, 1, 20, 1]),
    "per_pixel": ([8, 6, 20, 2], [8, 6, 1, 2]),
    "both_sides": ([1, 1, 20, 2], [8, 6, 20, 1]),
    "rank2_row": ([48, 5], [48, 1]),
    "scalar_like": ([7, 3, 17, 1], [1, 1, 1, 1]),
}


@pytest.mark.parametrize("dtype", ["u8", "f32"])
@pytest.mark.parametrize("name", sorted(BROADCAST_SHAPES))
def test_add_broadcast_matches_oracle(oracle_lib, product_lib, name, dtype):
    """numpy-style broadcasting of Add (equal ranks, ones repeat), quantized and float32."""
    da, db = BROADCAST_SHAPES[name]
    def build(g, rng):
        if dtype == "u8":
            a = g.tensor(B.DT_UINT8, da, B.ATTR_INPUT, scale=0.02, zero_point=128)
            b = g.tensor(B.DT_UINT8, db, B.ATTR_INPUT, scale=0.035, zero_point=117)
            y = g.tensor(B.DT_UINT8, [], B.ATTR_OUTPUT, scale=0.05, zero_point=120)
            av = rng.integers(0, 256, size=da[::-1]).astype(np.uint8)
            bv = rng.integers(0, 256, size=db[::-1]).astype(np.uint8)
        else:
            a = g.tensor(B.DT_FLOAT32, da, B.ATTR_INPUT)
            b = g.tensor(B.DT_FLOAT32, db, B.ATTR_INPUT)
            y = g.tensor(B.DT_FLOAT32, [], B.ATTR_OUTPUT)
            av = rng.standard_normal(da[::-1]).astype(np.float32)
            bv = rng.standard_normal(db[::-1]).astype(np.float32)
        g.add(a, b, y)
        return [(a, av), (b, bv)], [y]
    want, _ = G.run_case(oracle_lib, build, seed=4)
    got, kernels = G.run_case(product_lib, build, seed=4)
    assert any(k["name"] == "add_broadcast" for k in kernels), [k["name"] for k in kernels]
    assert want[0].shape == tuple(max(x, y) for x, y in zip(da, db))[::-1]
    G.assert_same(want, got)


def conv_then_add(W, H, C, N, k, Oc, swap=False, w_kind="s8pc", in_q=(0.02, 0), conv_q=(0.04, 131), res_q=(0.03, 7),
                  out_q=(0.06, 0), relu=True, dtype=B.DT_UINT8, stride=1):
    """x -> Conv2d -> t; Add(t, r) [operands swapped on request] -> Relu -> y, with r a second graph input."""
    def build(g, rng):
        x = g.tensor(dtype, [W, H, C, N], B.ATTR_INPUT, scale=in_q[0], zero_point=in_q[1])
        wshape = [k, k, C, Oc]
        if w_kind == "s8pc":
            ws = rng.uniform(0.001, 0.01, Oc).astype(np.float32)
            w = g.tensor(B.DT_INT8, wshape, B.ATTR_CONSTANT, scales=ws, channel_dim=3,
                         data=rng.integers(-127, 128, size=wshape[::-1]).astype(np.int8))
            bq = dict(scales=np.float32(in_q[0]) * ws, channel_dim=0)
        else:
            w = g.tensor(B.DT_UINT8, wshape, B.ATTR_CONSTANT, scale=0.01, zero_point=int(rng.integers(100, 157)),
                         data=rng.integers(0, 256, size=wshape[::-1]).astype(np.uint8))
            bq = dict(scale=float(np.float32(in_q[0]) * np.float32(0.01)), zero_point=0)
        b = g.tensor(B.DT_INT32, [Oc], B.ATTR_CONSTANT, data=rng.integers(-1000, 1001, size=Oc).astype(np.int32), **bq)
        t = g.tensor(dtype, [], B.ATTR_TRANSIENT, scale=conv_q[0], zero_point=conv_q[1])
        g.conv2d(x, w, b, t, stride=(stride, stride), pad_type=B.PAD_SAME)
        Wo, Ho = (W + stride - 1) // stride, (H + stride - 1) // stride
        r = g.tensor(dtype, [Wo, Ho, Oc, N], B.ATTR_INPUT, scale=res_q[0], zero_point=res_q[1])
        s_ = g.tensor(dtype, [], B.ATTR_TRANSIENT if relu else B.ATTR_OUTPUT, scale=out_q[0], zero_point=out_q[1])
        if swap:
            g.add(r, t, s_)
        else:
            g.add(t, r, s_)
        y = s_
        if relu:
            y = g.tensor(dtype, [], B.ATTR_OUTPUT, scale=out_q[0], zero_point=out_q[1])
            g.relu(s_, y)
        lo, hi = (0, 256) if dtype == B.DT_UINT8 else (-128, 128)
        np_t = B.NP_DTYPE[dtype]
        return [(x, rng.integers(lo, hi, size=(N, C, H, W)).astype(np_t)),
                (r, rng.integers(lo, hi, size=(N, Oc, Ho, Wo)).astype(np_t))], [y]
    return build


FUSED_ADD_CASES = {
    "expand_1x1": conv_then_add(14, 14, 64, 2, 1, 256),
    "expand_1x1_swapped": conv_then_add(14, 14, 64, 2, 1, 256, swap=True),
    "conv3x3_zp_border": conv_then_add(13, 11, 32, 2, 3, 48, in_q=(0.02, 128)),
    "u8_weights_linear": conv_then_add(9, 9, 96, 3, 1, 24, w_kind="u8", in_q=(0.03, 0), relu=False, out_q=(0.05, 120)),
    "stride2_3x3": conv_then_add(16, 16, 32, 1, 3, 64, stride=2),
    "int8_everything": conv_then_add(10, 10, 16, 2, 1, 32, dtype=B.DT_INT8, in_q=(0.05, -3), conv_q=(0.1, 4), res_q=(0.08, -9),
                                     out_q=(0.15, -128)),
    "oc_300_two_tiles": conv_then_add(7, 7, 64, 2, 1, 300),
    # more than eight tiles per SM with a short K: tiles of 65-128 columns go one per warp group, the residual's pieces
    # loaded by the epilogue threads themselves
    "many_tiles_64_96": conv_then_add(448, 400, 64, 1, 1, 96),
    "many_tiles_32_112_u8w": conv_then_add(448, 360, 32, 1, 1, 112, w_kind="u8", in_q=(0.03, 0)),
}


@pytest.mark.parametrize("name", sorted(FUSED_ADD_CASES))
def test_residual_add_fused_into_conv_matches_oracle(oracle_lib, product_lib, name):
    """Conv2d -> Add(-> Relu): the Add runs in the convolution's epilogue through its 64 KB table; the same
    graph with the fusion switched off and the oracle must give the same bytes."""
    os.environ.pop("B2VX_CONV_KERNEL", None)
    want, _ = G.run_case(oracle_lib, FUSED_ADD_CASES[name], seed=31)
    got, kernels = G.run_case(product_lib, FUSED_ADD_CASES[name], seed=31)
    names = [k["name"] for k in kernels]
    assert any("+add" in n for n in names) and not any(n.startswith("add_q") for n in names), names
    G.assert_same(want, got)
    os.environ["B2VX_FUSE_ADD"] = "0"
    try:
        unfused, kernels2 = G.run_case(product_lib, FUSED_ADD_CASES[name], seed=31)
    finally:
        os.environ.pop("B2VX_FUSE_ADD", None)
    assert any(k["name"].startswith("add_q") for k in kernels2)
    G.assert_same(want, unfused)


def test_add_int8_matches_oracle(oracle_lib, product_lib):
    def build(g, rng):
        n = 65536
        a = g.tensor(B.DT_INT8, [n], B.ATTR_INPUT, scale=0.03, zero_point=-5)
        b = g.tensor(B.DT_INT8, [n], B.ATTR_INPUT, scale=0.021, zero_point=17)
        y = g.tensor(B.DT_INT8, [], B.ATTR_OUTPUT, scale=0.04, zero_point=-20)
        g.add(a, b, y)
        i = np.arange(n)
        return [(a, (i >> 8).astype(np.uint8).view(np.int8)), (b, (i & 255).astype(np.uint8).view(np.int8))], [y]
    want, _ = G.run_case(oracle_lib, build, seed=1)
    for kernel in ("lut", "alu"):
        os.environ["B2VX_ADD_KERNEL"] = kernel
        try:
            got, _ = G.run_case(product_lib, build, seed=1)
        finally:
            os.environ.pop("B2VX_ADD_KERNEL", None)
        G.assert_same(want, got)


def test_add_int32_matches_oracle(oracle_lib, product_lib):
    """INT32 + INT32 as the reference's platform sample adds them (samples/platform_sample/platform_sample.cc:36-47),
    plain and with quantization parameters; values near the int32 limits saturate."""
    def case(quant):
        def build(g, rng):
            n = 4099
            kw = [dict(scale=0.5, zero_point=3), dict(scale=0.25, zero_point=-7), dict(scale=0.125, zero_point=11)] if quant else [{}, {}, {}]
            a = g.tensor(B.DT_INT32, [n], B.ATTR_INPUT, **kw[0])
            b = g.tensor(B.DT_INT32, [n], B.ATTR_INPUT, **kw[1])
            y = g.tensor(B.DT_INT32, [], B.ATTR_OUTPUT, **kw[2])
            g.add(a, b, y)
            av = rng.integers(-100000, 100000, size=n).astype(np.int32)
            bv = rng.integers(-100000, 100000, size=n).astype(np.int32)
            av[:4] = [2147483647, -2147483648, 2147483000, 5]
            bv[:4] = [2147483647, -2147483648, 1000, -5]
            return [(a, av), (b, bv)], [y]
        return build
    for quant in (False, True):
        want, _ = G.run_case(oracle_lib, case(quant), seed=4)
        got, kernels = G.run_case(product_lib, case(quant), seed=4)
        assert "add_i32" in [k["name"] for k in kernels]
        G.assert_same(want, got)


@pytest.mark.parametrize("group,w_kind", [(2, "s8pc"), (4, "u8"), (8, "s8pc")])
def test_grouped_conv_matches_oracle(oracle_lib, product_lib, group, w_kind):
    """ops::GroupedConv2d: kernel [3, 3, C/group, Oc]; the CUDA library runs it as a block-diagonal dense convolution."""
    C, Oc, W, H, N = 32, 48, 13, 11, 2

    def build(g, rng):
        x = g.tensor(B.DT_UINT8, [W, H, C, N], B.ATTR_INPUT, scale=0.02, zero_point=121)
        if w_kind == "s8pc":
            ws = rng.uniform(0.002, 0.01, Oc).astype(np.float32)
            w = g.tensor(B.DT_INT8, [3, 3, C // group, Oc], B.ATTR_CONSTANT, scales=ws, channel_dim=3,
                         data=rng.integers(-127, 128, size=(Oc, C // group, 3, 3)).astype(np.int8))
            b = g.tensor(B.DT_INT32, [Oc], B.ATTR_CONSTANT, scales=np.float32(0.02) * ws, channel_dim=0,
                         data=rng.integers(-800, 800, size=Oc).astype(np.int32))
        else:
            w = g.tensor(B.DT_UINT8, [3, 3, C // group, Oc], B.ATTR_CONSTANT, scale=0.01, zero_point=117,
                         data=rng.integers(0, 256, size=(Oc, C // group, 3, 3)).astype(np.uint8))
            b = g.tensor(B.DT_INT32, [Oc], B.ATTR_CONSTANT, scale=0.02 * 0.01, zero_point=0,
                         data=rng.integers(-800, 800, size=Oc).astype(np.int32))
        y = g.tensor(B.DT_UINT8, [], B.ATTR_OUTPUT, scale=0.06, zero_point=100)
        g.conv2d(x, w, b, y, pad_type=B.PAD_SAME, group=group)
        return [(x, rng.integers(0, 256, size=(N, C, H, W)).astype(np.uint8))], [y]
    want, _ = G.run_case(oracle_lib, build, seed=13)
    got, _ = G.run_case(product_lib, build, seed=13)
    G.assert_same(want, got)
    assert len(np.unique(want[0])) > 20


def test_softmax_matches_oracle(oracle_lib, product_lib):
    for build in (G.softmax_q(10, 7), G.softmax_q(1000, 3, beta=0.5)):
        want, _ = G.run_case(oracle_lib, build, seed=2)
        got, _ = G.run_case(product_lib, build, seed=2)
        G.assert_same(want, got, float_tol=SOFTMAX_TOL)


@pytest.mark.parametrize("batch", [1, 16])
def test_lenet_matches_oracle(oracle_lib, product_lib, conv_kernel, batch):
    want, _ = G.run_case(oracle_lib, G.lenet_synthetic(batch), seed=77)
    got, _ = G.run_case(product_lib, G.lenet_synthetic(batch), seed=77)
    G.assert_same(want[:1], got[:1])                       # uint8 logits: bit-exact
    G.assert_same(want[1:], got[1:], float_tol=SOFTMAX_TOL)  # float32 probabilities


def test_errors_are_reported_not_swallowed(product_lib):
    g = B.Graph(product_lib)
    x = g.tensor(B.DT_UINT8, [4, 4, 8, 1], B.ATTR_INPUT, scale=0.1, zero_point=0)
    w = g.tensor(B.DT_UINT8, [3, 3, 4, 8], B.ATTR_CONSTANT, scale=0.1, zero_point=0,
                 data=np.zeros((8, 4, 3, 3), np.uint8))   # Ic 4 != C 8
    y = g.tensor(B.DT_UINT8, [], B.ATTR_OUTPUT, scale=0.1, zero_point=0)
    g.conv2d(x, w, None, y, pad_type=B.PAD_SAME)
    with pytest.raises(B.B2vxError) as e:
        g.compile()
    assert e.value.status == 3  # SHAPE_MISMATCH
    g.close()
