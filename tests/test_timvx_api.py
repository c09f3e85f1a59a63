"""The tim::vx C++ surface as user code sees it: a LeNet program written against the public
headers only is compiled and run on the CPU oracle build (CPU test) and on the CUDA build (GPU
test); the two must print the same uint8 logits, and probabilities within 1e-5."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC = os.path.join(ROOT, "tests", "cpp", "lenet_api.cc")


def build(tmp_path, libdir, libs, name):
    exe = str(tmp_path / name)
    cmd = ["/usr/bin/g++", "-std=c++17", "-O1", "-Wall", "-Wextra", "-Werror", "-I" + os.path.join(ROOT, "include"), SRC,
           "-L" + libdir] + ["-l" + l for l in libs] + ["-Wl,-rpath," + libdir, "-o", exe]
    subprocess.check_call(cmd)
    return exe


def run(exe, batch):
    out = subprocess.run([exe, str(batch)], capture_output=True, text=True, timeout=300, env=dict(os.environ, VSI_NN_LOG_LEVEL="1"))
    assert out.returncode == 0, out.stdout + out.stderr
    rows = []
    for line in out.stdout.strip().splitlines():
        f = line.split()
        rows.append(([int(v) for v in f[1:11]], [float(v) for v in f[12:22]]))
    assert len(rows) == batch
    return rows


def oracle_exe(tmp_path, oracle_lib):
    return build(tmp_path, os.path.join(ROOT, "oracle", "_build"), ["tim-vx-oracle", "b2vx_oracle"], "lenet_oracle")


def test_user_program_compiles_and_runs_on_the_oracle(tmp_path, oracle_lib):
    rows = run(oracle_exe(tmp_path, oracle_lib), 3)
    for logits, prob in rows:
        assert abs(sum(prob) - 1.0) < 1e-3
        assert len(set(logits)) > 1   # not a constant output


@pytest.mark.gpu
def test_user_program_on_gpu_matches_oracle(tmp_path, oracle_lib, product_lib):
    want = run(oracle_exe(tmp_path, oracle_lib), 4)
    exe = build(tmp_path, os.path.join(ROOT, "tim-vx_b200", "csrc"), ["tim-vx", "b2vx"], "lenet_gpu")
    got = run(exe, 4)
    for (wl, wp), (gl, gp) in zip(want, got):
        assert wl == gl
        assert max(abs(a - b) for a, b in zip(wp, gp)) <= 2e-5
