"""Reshape, Transpose, Concat and DataConvert: the nodes the reference's exported graphs put between the
compute nodes (samples/multi_device/vx_mobilenet.cc:570-571,832-840; vx_resnet50.cc:1347-1349).

CPU tests: the oracle against numpy (a WHCN shape [d0, d1, ...] is the numpy shape reversed), and a C++
program written against the public headers (tests/cpp/movement_ops.cc) on the oracle build.
GPU tests: the CUDA library against the oracle, bit for bit, through the C ABI, and the same C++ program on
the CUDA build printing the same line as on the oracle build.
"""
import itertools
import os
import subprocess

import numpy as np
import pytest

import graph_cases as G
import pyb2vx as B

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC = os.path.join(ROOT, "tests", "cpp", "movement_ops.cc")

NP = {B.DT_UINT8: np.uint8, B.DT_INT8: np.int8, B.DT_FLOAT32: np.float32, B.DT_INT32: np.int32}


def _data(rng, dtype, dims):
    shape = tuple(reversed(dims))
    if dtype == B.DT_FLOAT32:
        return rng.uniform(-4, 4, size=shape).astype(np.float32)
    if dtype == B.DT_INT32:
        return rng.integers(-100000, 100000, size=shape).astype(np.int32)
    info = np.iinfo(NP[dtype])
    return rng.integers(info.min, info.max + 1, size=shape).astype(NP[dtype])


def _q(dtype, scale=0.1, zp=3):
    return dict(scale=scale, zero_point=zp) if dtype in (B.DT_UINT8, B.DT_INT8) else {}


def transpose_case(dtype, dims, perm):
    def build(g, rng):
        x = g.tensor(dtype, dims, B.ATTR_INPUT, **_q(dtype))
        y = g.tensor(dtype, [], B.ATTR_OUTPUT, **_q(dtype))
        g.transpose(x, y, perm)
        return [(x, _data(rng, dtype, dims))], [y]
    return build


def reshape_case(dtype, dims, new_dims):
    def build(g, rng):
        x = g.tensor(dtype, dims, B.ATTR_INPUT, **_q(dtype))
        y = g.tensor(dtype, [], B.ATTR_OUTPUT, **_q(dtype))
        g.reshape(x, y, new_dims)
        return [(x, _data(rng, dtype, dims))], [y]
    return build


def concat_case(dtype, dims_list, axis, quants=None, out_q=None):
    def build(g, rng):
        ins = []
        for k, dims in enumerate(dims_list):
            q = quants[k] if quants else (0.1, 3)
            x = g.tensor(dtype, dims, B.ATTR_INPUT, **_q(dtype, *q))
            ins.append((x, _data(rng, dtype, dims)))
        y = g.tensor(dtype, [], B.ATTR_OUTPUT, **_q(dtype, *(out_q or (0.1, 3))))
        g.concat([x for x, _ in ins], y, axis)
        return ins, [y]
    return build


def convert_case(in_dtype, out_dtype, dims, in_q=(0.1, 3), out_q=(0.07, 100)):
    def build(g, rng):
        x = g.tensor(in_dtype, dims, B.ATTR_INPUT, **_q(in_dtype, *in_q))
        y = g.tensor(out_dtype, [], B.ATTR_OUTPUT, **_q(out_dtype, *out_q))
        g.dataconvert(x, y)
        data = _data(rng, in_dtype, dims)
        if in_dtype == B.DT_FLOAT32:
            data = (data * 5).astype(np.float32)      # reaches both saturation ends of the 8-bit output
            data.reshape(-1)[:4] = [0.035, 0.105, -0.035, 1e9]   # ties of real / 0.07 and a saturating value
        return [(x, data)], [y]
    return build


CASES = {}
for _perm in itertools.permutations(range(4)):
    CASES["transpose_u8_%d%d%d%d" % _perm] = transpose_case(B.DT_UINT8, [5, 4, 3, 2], list(_perm))
CASES.update({
    "transpose_u8_nhwc_image": transpose_case(B.DT_UINT8, [3, 32, 24, 2], [1, 2, 0, 3]),
    "transpose_f32_rank3": transpose_case(B.DT_FLOAT32, [7, 5, 3], [2, 0, 1]),
    # large enough in both contiguous dimensions for the tiled byte transpose, with ragged tile edges
    "transpose_u8_tiled_wh": transpose_case(B.DT_UINT8, [40, 50, 3, 2], [1, 0, 2, 3]),
    "transpose_u8_tiled_nhwc64": transpose_case(B.DT_UINT8, [64, 19, 21, 2], [1, 2, 0, 3]),
    "transpose_u8_tiled_rank2": transpose_case(B.DT_UINT8, [257, 131], [1, 0]),
    "transpose_i32_rank2": transpose_case(B.DT_INT32, [1, 3], [1, 0]),
    "transpose_s8_rank2": transpose_case(B.DT_INT8, [33, 17], [1, 0]),
    "reshape_u8_4d_to_2d": reshape_case(B.DT_UINT8, [5, 4, 3, 2], [60, 2]),
    "reshape_u8_4d_to_4d": reshape_case(B.DT_UINT8, [5, 4, 3, 2], [2, 10, 3, 2]),
    "reshape_u8_logits": reshape_case(B.DT_UINT8, [1, 1, 1001, 2], [1001, 2]),
    "reshape_f32_2d_to_3d": reshape_case(B.DT_FLOAT32, [24, 3], [4, 6, 3]),
    "reshape_i32_1d": reshape_case(B.DT_INT32, [16], [16]),
    "concat_u8_axis0": concat_case(B.DT_UINT8, [[3, 4, 5, 2], [6, 4, 5, 2]], 0),
    "concat_u8_axis1": concat_case(B.DT_UINT8, [[3, 4, 5, 2], [3, 1, 5, 2], [3, 2, 5, 2]], 1),
    "concat_u8_axis2_ragged": concat_case(B.DT_UINT8, [[6, 4, 5, 2], [6, 4, 20, 2]], 2),
    "concat_u8_axis2_channels16": concat_case(B.DT_UINT8, [[7, 7, 32, 2], [7, 7, 16, 2], [7, 7, 64, 2]], 2),
    "concat_u8_axis3": concat_case(B.DT_UINT8, [[3, 4, 5, 2], [3, 4, 5, 1]], 3),
    "concat_u8_requant": concat_case(B.DT_UINT8, [[7, 7, 32, 2], [7, 7, 16, 2]], 2, quants=[(0.05, 7), (0.031, 120)], out_q=(0.04, 60)),
    "concat_f32_rank2": concat_case(B.DT_FLOAT32, [[10, 3], [7, 3]], 0),
    "convert_u8_to_u8": convert_case(B.DT_UINT8, B.DT_UINT8, [9, 5, 20, 2]),
    "convert_s8_to_u8": convert_case(B.DT_INT8, B.DT_UINT8, [33, 3], in_q=(0.5, -1)),
    "convert_f32_to_u8": convert_case(B.DT_FLOAT32, B.DT_UINT8, [6, 5, 3, 2]),
    "convert_u8_to_f32": convert_case(B.DT_UINT8, B.DT_FLOAT32, [6, 5, 3, 2]),
})


def test_oracle_matches_numpy(oracle_lib):
    rng = np.random.default_rng(3)
    # transpose: output dimension i is input dimension perm[i]; numpy axes run the other way round
    for perm in itertools.permutations(range(4)):
        dims = [5, 4, 3, 2]
        out, _ = G.run_case(oracle_lib, transpose_case(B.DT_UINT8, dims, list(perm)), seed=3)
        x = _data(np.random.default_rng(3), B.DT_UINT8, dims)
        axes = [3 - perm[3 - k] for k in range(4)]
        assert np.array_equal(out[0], x.transpose(axes)), perm
    out, _ = G.run_case(oracle_lib, reshape_case(B.DT_UINT8, [5, 4, 3, 2], [2, 10, 3, 2]), seed=4)
    x = _data(np.random.default_rng(4), B.DT_UINT8, [5, 4, 3, 2])
    assert np.array_equal(out[0], x.reshape(2, 3, 10, 2))
    out, _ = G.run_case(oracle_lib, concat_case(B.DT_UINT8, [[3, 4, 5, 2], [3, 1, 5, 2], [3, 2, 5, 2]], 1), seed=5)
    r = np.random.default_rng(5)
    parts = [_data(r, B.DT_UINT8, d) for d in ([3, 4, 5, 2], [3, 1, 5, 2], [3, 2, 5, 2])]
    assert np.array_equal(out[0], np.concatenate(parts, axis=2))
    # requantizing concat and DataConvert: dequantize, divide, round half to even, add zero point, clamp
    out, _ = G.run_case(oracle_lib, convert_case(B.DT_UINT8, B.DT_UINT8, [9, 5, 20, 2]), seed=6)
    x = _data(np.random.default_rng(6), B.DT_UINT8, [9, 5, 20, 2])
    real = (x.astype(np.float32) - np.float32(3)) * np.float32(0.1)
    want = np.clip(np.rint(real / np.float32(0.07)) + 100, 0, 255).astype(np.uint8)
    assert np.array_equal(out[0], want)
    del rng


@pytest.mark.gpu
@pytest.mark.parametrize("name", sorted(CASES))
def test_gpu_matches_oracle(oracle_lib, product_lib, name):
    want, _ = G.run_case(oracle_lib, CASES[name], seed=21)
    got, kernels = G.run_case(product_lib, CASES[name], seed=21)
    G.assert_same(want, got)
    if name == "concat_u8_axis2_channels16":
        assert [k["name"] for k in kernels if k["name"].startswith("concat")] == ["concat_c16"] * 3


@pytest.mark.gpu
def test_mobilenet_style_head_and_tail_on_gpu(oracle_lib, product_lib):
    """NHWC image -> Transpose -> Conv2d ... Pool2d -> Transpose -> Reshape -> Softmax, as in the exported MobileNet."""
    def build(g, rng):
        x = g.tensor(B.DT_UINT8, [3, 32, 32, 2], B.ATTR_INPUT, scale=0.0078125, zero_point=128)
        t = g.tensor(B.DT_UINT8, [], B.ATTR_TRANSIENT, scale=0.0078125, zero_point=128)
        g.transpose(x, t, [1, 2, 0, 3])
        w = g.tensor(B.DT_UINT8, [3, 3, 3, 24], B.ATTR_CONSTANT, scale=0.02, zero_point=120,
                     data=rng.integers(0, 256, size=(24, 3, 3, 3)).astype(np.uint8))
        b = g.tensor(B.DT_INT32, [24], B.ATTR_CONSTANT, scale=0.0078125 * 0.02, zero_point=0,
                     data=rng.integers(-500, 500, size=24).astype(np.int32))
        c = g.tensor(B.DT_UINT8, [], B.ATTR_TRANSIENT, scale=0.05, zero_point=0)
        g.conv2d(t, w, b, c, stride=(2, 2), pad_type=B.PAD_SAME)
        p = g.tensor(B.DT_UINT8, [], B.ATTR_TRANSIENT, scale=0.05, zero_point=0)
        g.pool2d(c, p, B.POOL_AVG, (16, 16), (16, 16))
        u = g.tensor(B.DT_UINT8, [], B.ATTR_TRANSIENT, scale=0.05, zero_point=0)
        g.transpose(p, u, [2, 0, 1, 3])
        r = g.tensor(B.DT_UINT8, [], B.ATTR_TRANSIENT, scale=0.05, zero_point=0)
        g.reshape(u, r, [24, 2])
        y = g.tensor(B.DT_FLOAT32, [], B.ATTR_OUTPUT)
        g.softmax(r, y, beta=1.0, axis=0)
        return [(x, rng.integers(0, 256, size=(2, 32, 32, 3)).astype(np.uint8))], [y]
    want, _ = G.run_case(oracle_lib, build, seed=9)
    got, _ = G.run_case(product_lib, build, seed=9)
    G.assert_same(want, got, float_tol=1e-5)


def _build(tmp_path, libdir, libs, name):
    exe = str(tmp_path / name)
    subprocess.check_call(["/usr/bin/g++", "-std=c++17", "-O1", "-Wall", "-Wextra", "-Werror", "-I" + os.path.join(ROOT, "include"), SRC,
                           "-L" + libdir] + ["-l" + l for l in libs] + ["-Wl,-rpath," + libdir, "-o", exe])
    return exe


def _run(exe):
    out = subprocess.run([exe], capture_output=True, text=True, timeout=300, env=dict(os.environ, VSI_NN_LOG_LEVEL="1"))
    assert out.returncode == 0, "exit %d\n%s%s" % (out.returncode, out.stdout, out.stderr)
    lines = out.stdout.strip().splitlines()
    assert lines[-1] == "ok movement ops"
    return [l for l in lines if l.startswith("out ")][0]


def test_cpp_program_on_the_oracle(tmp_path, oracle_lib):
    _run(_build(tmp_path, os.path.join(ROOT, "oracle", "_build"), ["tim-vx-oracle", "b2vx_oracle"], "movement_oracle"))


@pytest.mark.gpu
def test_cpp_program_on_gpu_matches_oracle(tmp_path, oracle_lib, product_lib):
    want = _run(_build(tmp_path, os.path.join(ROOT, "oracle", "_build"), ["tim-vx-oracle", "b2vx_oracle"], "movement_oracle"))
    got = _run(_build(tmp_path, os.path.join(ROOT, "tim-vx_b200", "csrc"), ["tim-vx", "b2vx"], "movement_gpu"))
    assert got == want
