"""Batch sharding across ranks, exercised on CPU with the gloo backend (world size 2).

Each rank runs its shard of a batch through a replica of the same seeded network
(the oracle-backed build of tim-vx_b200/samples), the outputs are gathered, and
the result must equal the single-process run of the whole batch bit for bit:
images are independent, so sharding by batch changes nothing.
"""
import ctypes as C
import os
import subprocess
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = r'''
import ctypes as C, os, sys
import numpy as np
import torch.distributed as dist
sys.path.insert(0, os.path.join(sys.argv[1], "tim-vx_b200")); sys.path.insert(0, sys.argv[1])
import bench, sharding
dist.init_process_group("gloo")
rank, world = dist.get_rank(), dist.get_world_size()
total = int(sys.argv[2])
lib = bench.load_samples(bench.SAMPLES_ORACLE_LIB)
# every rank derives the same full input, then keeps its own shard
full = lib.b2vx_net_create(b"lenet", total, 11, 0)
x = np.empty(lib.b2vx_net_input_bytes(full), np.uint8)
lib.b2vx_net_synthetic_input(full, 3, x.ctypes.data)
b, e = sharding.shard_range(total, rank, world)
lo, hi = sharding.shard_bytes(x.nbytes, total, rank, world)
net = lib.b2vx_net_create(b"lenet", e - b, 11, 0)
xs = np.ascontiguousarray(x[lo:hi])
assert lib.b2vx_net_set_input(net, xs.ctypes.data) == 0 and lib.b2vx_net_run(net) == 0
y = np.empty(lib.b2vx_net_output_bytes(net), np.uint8)
assert lib.b2vx_net_get_output(net, y.ctypes.data) == 0
out = sharding.gather_outputs(y.reshape(e - b, 10), total, dist)
slowest = sharding.max_over_ranks(1.0 + rank, dist)
if rank == 0:
    np.save(sys.argv[3], out)
    assert slowest == float(world)
dist.destroy_process_group()
'''


def test_shard_range_covers_everything():
    sys.path.insert(0, os.path.join(ROOT, "tim-vx_b200"))
    import sharding
    for n in (1, 7, 64, 1000):
        for world in (1, 2, 3, 8):
            spans = [sharding.shard_range(n, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [e - b for b, e in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        sharding.shard_range(4, 4, 4)


def test_two_ranks_equal_one_process(tmp_path, oracle_lib):
    sys.path.insert(0, ROOT)
    import bench
    total = 5   # odd on purpose: ranks get 3 and 2 images
    lib = bench.load_samples(bench.SAMPLES_ORACLE_LIB)
    net = lib.b2vx_net_create(b"lenet", total, 11, 0)
    x = np.empty(lib.b2vx_net_input_bytes(net), np.uint8)
    lib.b2vx_net_synthetic_input(net, 3, x.ctypes.data)
    assert lib.b2vx_net_set_input(net, x.ctypes.data) == 0 and lib.b2vx_net_run(net) == 0
    want = np.empty(lib.b2vx_net_output_bytes(net), np.uint8)
    assert lib.b2vx_net_get_output(net, want.ctypes.data) == 0
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    out = tmp_path / "out.npy"
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29531", str(script), ROOT, str(total), str(out)]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    got = np.load(out)
    assert np.array_equal(got.reshape(-1), want)
