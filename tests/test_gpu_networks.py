"""Whole networks built through the tim::vx API (tim-vx_b200/samples): CUDA output vs CPU oracle
output on the same seeded weights and inputs, bit for bit.  Also a spread check on the oracle side so
that "equal" cannot mean "all saturated"."""
import os
import subprocess
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
RUN = os.path.join(ROOT, "tests", "run_net.py")


def run(backend, net, batch, tmp_path, env=None):
    out = str(tmp_path / ("%s_%s_%d.npy" % (backend, net, batch)))
    e = dict(os.environ)
    e.update(env or {})
    r = subprocess.run([sys.executable, RUN, backend, net, str(batch), "7", "9", out], capture_output=True, text=True,
                       timeout=900, env=e)
    assert r.returncode == 0, r.stdout[-1500:] + r.stderr[-1500:]
    return np.load(out)


def test_oracle_network_outputs_have_spread(tmp_path, oracle_lib):
    y = run("oracle", "mobilenetv2", 1, tmp_path)
    assert len(np.unique(y)) > 10 and y.min() > 0 and y.max() < 255


@pytest.mark.gpu
@pytest.mark.parametrize("net,batch", [("lenet", 3), ("resnet50", 2), ("mobilenetv2", 2)])
def test_network_matches_oracle(tmp_path, oracle_lib, product_lib, net, batch):
    want = run("oracle", net, batch, tmp_path)
    got = run("gpu", net, batch, tmp_path)
    bad = np.flatnonzero(want != got)
    assert bad.size == 0, "%d of %d outputs differ (first %d: oracle %d gpu %d)" % (
        bad.size, want.size, bad[0], want[bad[0]], got[bad[0]])
    if net != "lenet":
        assert len(np.unique(want)) > 10


@pytest.mark.gpu
def test_resnet50_cuda_core_path_matches_too(tmp_path, oracle_lib, product_lib):
    """The CUDA-core convolution path on the same network: an independent GPU implementation
    that must land on the same bytes as the tensor-core path and the oracle."""
    want = run("oracle", "resnet50", 1, tmp_path)
    got = run("gpu", "resnet50", 1, tmp_path, env={"B2VX_CONV_KERNEL": "simt"})
    assert np.array_equal(want, got)
