"""The benchmark configurations at their full sizes, checked through properties that do not need the
CPU oracle to chew through the whole workload:

* batch independence: images are independent, the synthetic input of a small batch is a prefix of the
  large batch's input, so the first images of a full-size run must equal the oracle's small-batch run;
* rows of a FullyConnected are independent: the oracle on the first rows pins the full-size GEMM;
* elementwise: the oracle on a prefix, and the two Add kernels against each other on everything;
* the tensor-core and the CUDA-core convolution paths are independent implementations: their outputs
  over the full batch must be the same bytes.
"""
import os
import subprocess
import sys

import numpy as np
import pytest

import pyb2vx as B
import opworkloads

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
RUN = os.path.join(ROOT, "tests", "run_net.py")
pytestmark = pytest.mark.gpu


def run_net(backend, net, batch, tmp_path, env=None, tag=""):
    out = str(tmp_path / ("%s_%s_%d%s.npy" % (backend, net, batch, tag)))
    e = dict(os.environ)
    e.update(env or {})
    r = subprocess.run([sys.executable, RUN, backend, net, str(batch), "7", "9", out], capture_output=True, text=True,
                       timeout=1200, env=e)
    assert r.returncode == 0, r.stdout[-1500:] + r.stderr[-1500:]
    return np.load(out)


@pytest.mark.parametrize("net,full,small", [("resnet50", 64, 3), ("mobilenetv2", 64, 3), ("lenet", 256, 16)])
def test_full_batch_prefix_matches_oracle(tmp_path, oracle_lib, product_lib, net, full, small):
    want = run_net("oracle", net, small, tmp_path)
    got = run_net("gpu", net, full, tmp_path)
    per_image = got.size // full
    assert want.size == small * per_image
    assert np.array_equal(got[:small * per_image], want)
    # and the rest of the batch is not a copy of it: different images, different logits
    assert not np.array_equal(got[:per_image], got[per_image:2 * per_image])


def test_resnet50_full_batch_tensor_core_equals_cuda_core(tmp_path, product_lib):
    a = run_net("gpu", "resnet50", 64, tmp_path, tag="_tc")
    b = run_net("gpu", "resnet50", 64, tmp_path, env={"B2VX_CONV_KERNEL": "simt"}, tag="_simt")
    assert np.array_equal(a, b)


SWITCHES = [{"B2VX_TC_STORE": "tma"}, {"B2VX_TC_BRES": "0"}, {"B2VX_TC_TEAMS": "0"}, {"B2VX_FUSE_ADD": "0"},
            {"B2VX_PDL": "0", "B2VX_CUDA_GRAPH": "0"}, {"B2VX_TC_BN": "64"}, {"B2VX_POOL_2X2": "0"}, {"B2VX_TC_HALO": "0"}, {"B2VX_DW_STRIP": "0"}, {"B2VX_DW_PIPE": "1"}]


@pytest.mark.parametrize("net,batch", [("resnet50", 8), ("mobilenetv2", 8)])
def test_every_kernel_variant_gives_the_same_bytes(tmp_path, product_lib, net, batch):
    """The per-process switches select other code paths of the GEMM kernel (staged TMA stores, weights through the
    ring, one tile per sixteen epilogue warps, the Add as its own kernel, plain launches, narrow tiles): the
    network's output must not change by a byte."""
    want = run_net("gpu", net, batch, tmp_path)
    for k, env in enumerate(SWITCHES):
        got = run_net("gpu", net, batch, tmp_path, env=env, tag="_v%d" % k)
        assert np.array_equal(got, want), env


def _run_graph(lib, spec, batch, seed, inputs=None, env=None):
    old = {}
    for k, v in (env or {}).items():
        old[k] = os.environ.get(k)
        os.environ[k] = v
    try:
        g = B.Graph(lib)
        try:
            w = opworkloads.build(spec, batch, g, np.random.default_rng(seed))
            g.compile()
            arrays = inputs if inputs is not None else [a for _, a in w["inputs"]]
            for (tid, _), arr in zip(w["inputs"], arrays):
                g.write(tid, arr)
            g.run()
            return [g.read(t) for t in w["outputs"]], arrays, [k["name"] for k in g.kernels()]
        finally:
            g.close()
    finally:
        for k, v in old.items():
            if v is None:
                os.environ.pop(k, None)
            else:
                os.environ[k] = v


@pytest.mark.parametrize("n", [4096])
def test_full_size_gemm_rows_match_oracle(oracle_lib, product_lib, n):
    """gemm:n:n:n on the tensor cores; the oracle recomputes the first 48 rows from the same weights."""
    full, xs, kernels = _run_graph(product_lib, "gemm:%d:%d:%d" % (n, n, n), 1, seed=5)
    assert any(k.startswith("gemm_i8_tc") for k in kernels)
    rows = 48
    part, _, _ = _run_graph(oracle_lib, "gemm:%d:%d:%d" % (rows, n, n), 1, seed=5, inputs=[xs[0][:rows]])
    assert np.array_equal(full[0][:rows], part[0])
    assert len(np.unique(full[0])) > 50


@pytest.mark.parametrize("m", [4096, 4000])
def test_pair_mode_gemm_equals_one_tile_at_a_time(oracle_lib, product_lib, m):
    """K = 4096 with several tiles per CTA: two M tiles share every weight block (pair mode).  Same bytes as the kernel
    working on one tile at a time (B2VX_TC_PAIR=0), whole matrix, CTAs with odd and even tile counts and a ragged last
    M tile; the oracle on the first rows."""
    spec = "gemm:%d:4096:4096" % m
    pair, xs, kernels = _run_graph(product_lib, spec, 1, seed=12)
    assert any(k.startswith("gemm_i8_tc") for k in kernels)
    single, _, _ = _run_graph(product_lib, spec, 1, seed=12, inputs=xs, env={"B2VX_TC_PAIR": "0"})
    assert np.array_equal(pair[0], single[0])
    rows = 40
    part, _, _ = _run_graph(oracle_lib, "gemm:%d:4096:4096" % rows, 1, seed=12, inputs=[xs[0][:rows]])
    assert np.array_equal(pair[0][:rows], part[0])


def test_decode_like_gemm_matches_oracle(oracle_lib, product_lib):
    for m in (1, 16):
        spec = "gemm:%d:4096:4096" % m
        got, xs, _ = _run_graph(product_lib, spec, 1, seed=6)
        want, _, _ = _run_graph(oracle_lib, spec, 1, seed=6, inputs=xs)
        assert np.array_equal(got[0], want[0])


def test_full_size_conv_sweep_prefix_matches_oracle(oracle_lib, product_lib):
    """The 3x3 / 1x1 / stride-2 convolutions of the sweep at batch 256; the oracle on the first two images."""
    for spec in ("conv:3:64:64:56:1", "conv:1:64:64:56:1", "conv:3:64:64:56:2"):
        got, xs, kernels = _run_graph(product_lib, spec, 256, seed=8)
        assert any(k.startswith("gemm_i8_tc") for k in kernels)
        want, _, _ = _run_graph(oracle_lib, spec, 2, seed=8, inputs=[xs[0][:2]])
        assert np.array_equal(got[0][:2], want[0])


def test_full_size_conv_with_fused_residual_add_prefix_matches_oracle(oracle_lib, product_lib):
    """The tail of a bottleneck block (1x1 expand convolution, residual Add, Relu) at batch 256: one fused launch."""
    for spec in ("convadd:1:64:256:56:1", "convadd:3:64:64:56:1"):
        got, xs, kernels = _run_graph(product_lib, spec, 256, seed=10)
        assert any(k.startswith("gemm_i8_tc") and "+add" in k for k in kernels), kernels
        assert not any(k.startswith("add_q") for k in kernels), kernels
        want, _, _ = _run_graph(oracle_lib, spec, 2, seed=10, inputs=[x[:2] for x in xs])
        assert np.array_equal(got[0][:2], want[0])


def test_full_size_add_kernels_agree_and_prefix_matches_oracle(oracle_lib, product_lib):
    spec = "add:67108864"
    lut, xs, k1 = _run_graph(product_lib, spec, 1, seed=9, env={"B2VX_ADD_KERNEL": "lut"})
    alu, _, k2 = _run_graph(product_lib, spec, 1, seed=9, inputs=xs, env={"B2VX_ADD_KERNEL": "alu"})
    assert k1 == ["add_q_lut"] and k2 == ["add_q"]
    assert np.array_equal(lut[0], alu[0])
    rows = 4096                                   # 1 Mi elements
    want, _, _ = _run_graph(oracle_lib, "add:%d" % (rows * 256), 1, seed=9, inputs=[x[:rows] for x in xs])
    assert np.array_equal(lut[0][:rows], want[0])
