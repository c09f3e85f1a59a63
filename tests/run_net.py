"""Run one synthetic network (tim-vx_b200/samples) on the CUDA build or on the CPU oracle build and
save its uint8 output.  Each backend runs in its own process: both sample libraries export the same
symbols.  usage: run_net.py gpu|oracle <net> <batch> <weight seed> <input seed> <out.npy>"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import bench  # noqa: E402


def main():
    backend, net, batch, wseed, iseed, out = sys.argv[1], sys.argv[2], int(sys.argv[3]), int(sys.argv[4]), int(sys.argv[5]), sys.argv[6]
    lib = bench.load_samples(bench.SAMPLES_LIB if backend == "gpu" else bench.SAMPLES_ORACLE_LIB)
    h = lib.b2vx_net_create(net.encode(), batch, wseed, 0)
    assert h, "network creation failed"
    x = np.empty(lib.b2vx_net_input_bytes(h), np.uint8)
    lib.b2vx_net_synthetic_input(h, iseed, x.ctypes.data)
    assert lib.b2vx_net_set_input(h, x.ctypes.data) == 0
    assert lib.b2vx_net_run(h) == 0
    assert lib.b2vx_net_run(h) == 0   # a second run must give the same answer (no state carried over)
    y = np.empty(lib.b2vx_net_output_bytes(h), np.uint8)
    assert lib.b2vx_net_get_output(h, y.ctypes.data) == 0
    np.save(out, y)
    lib.b2vx_net_destroy(h)


if __name__ == "__main__":
    main()
