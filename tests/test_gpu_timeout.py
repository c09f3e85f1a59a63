"""The bounded waits of the tensor-core kernel, exercised without a GPU fault.

B2VX_TEST_STALL=1 (tim-vx_b200/csrc/gemm_tc.cu, gemm_tc_launch) makes the first GEMM launch of a process announce
16 bytes more than its loads deliver and shortens its wait limit to about a millisecond: every real load lands, one
barrier never completes, the waiting warp records a code in the status word, the CTAs leave through their common
exit.  Graph::Run must then report B2VX_DEVICE_TIMEOUT, and the same graph on the same context must run correctly
right afterwards.
"""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CHILD = r'''
import sys
sys.path.insert(0, %(root)r + "/tests"); sys.path.insert(0, %(root)r + "/tim-vx_b200")
import numpy as np
import graph_cases as G, oracle_paths as O, pyb2vx as B
build = G.conv2d_q(28, 28, 64, 2, 1, 1, 128)
want, _ = G.run_case(O.load(O.ORACLE_LIB), build, seed=4)
lib = B.load(B.PRODUCT_LIB)
g = B.Graph(lib, 0)
inputs, outputs = build(g, np.random.default_rng(4))
g.compile()
assert any(k["name"].startswith("gemm_i8_tc") for k in g.kernels())
for tid, arr in inputs:
    g.write(tid, arr)
try:
    g.run()
    print("FIRST_RUN_OK")
except B.B2vxError as e:
    print("FIRST_RUN_STATUS", e.status, str(e))
g.run()
got = [g.read(t) for t in outputs]
G.assert_same(want, got)
print("SECOND_RUN_MATCHES_ORACLE")
g.close()
'''


@pytest.mark.gpu
def test_a_wait_that_runs_out_is_reported_and_the_context_stays_usable(product_lib):
    env = dict(os.environ, B2VX_TEST_STALL="1", B2VX_CUDA_GRAPH="0")
    out = subprocess.run([sys.executable, "-c", CHILD % {"root": ROOT}], capture_output=True, text=True, env=env, timeout=300)
    assert out.returncode == 0, out.stdout + out.stderr
    assert "FIRST_RUN_STATUS 7" in out.stdout, out.stdout + out.stderr      # B2VX_DEVICE_TIMEOUT
    assert "gave up waiting on a barrier" in out.stdout
    assert "SECOND_RUN_MATCHES_ORACLE" in out.stdout, out.stdout + out.stderr
