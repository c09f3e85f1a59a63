"""tim::vx::platform (devices, executors, executables) and the serialised-graph round trip
(Graph::CompileToBinary -> ops::NBG): a C++ program written against the public headers runs on the
CPU oracle build (CPU test) and on the CUDA build (GPU test, every GPU of the box); inside the
program each executable's output must equal the plain graph's, and across builds the printed bytes
must be the same."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC = os.path.join(ROOT, "tests", "cpp", "platform_api.cc")


def build(tmp_path, libdir, libs, name):
    exe = str(tmp_path / name)
    cmd = ["/usr/bin/g++", "-std=c++17", "-O1", "-Wall", "-Wextra", "-Werror", "-I" + os.path.join(ROOT, "include"), SRC,
           "-L" + libdir] + ["-l" + l for l in libs] + ["-Wl,-rpath," + libdir, "-o", exe]
    subprocess.check_call(cmd)
    return exe


def run(exe):
    out = subprocess.run([exe], capture_output=True, text=True, timeout=300, env=dict(os.environ, VSI_NN_LOG_LEVEL="1"))
    assert out.returncode == 0, "exit %d\n%s%s" % (out.returncode, out.stdout, out.stderr)
    lines = out.stdout.strip().splitlines()
    assert lines[-1].startswith("ok ")
    return lines


def oracle_lines(tmp_path, oracle_lib):
    exe = build(tmp_path, os.path.join(ROOT, "oracle", "_build"), ["tim-vx-oracle", "b2vx_oracle"], "platform_oracle")
    return run(exe)


def test_platform_api_on_the_oracle(tmp_path, oracle_lib):
    lines = oracle_lines(tmp_path, oracle_lib)
    graph = [l for l in lines if l.startswith("graph ")][0].split()[2:]
    assert len(set(graph)) > 3                       # not a constant output
    dev = [l for l in lines if l.startswith("device ")]
    assert len(dev) == 1 and dev[0].split()[2:] == graph


@pytest.mark.gpu
def test_platform_api_on_gpu_matches_oracle(tmp_path, oracle_lib, product_lib):
    want = [l for l in oracle_lines(tmp_path, oracle_lib) if l.startswith("graph ")][0].split()[2:]
    exe = build(tmp_path, os.path.join(ROOT, "tim-vx_b200", "csrc"), ["tim-vx", "b2vx"], "platform_gpu")
    lines = run(exe)
    assert [l for l in lines if l.startswith("graph ")][0].split()[2:] == want
    dev = [l for l in lines if l.startswith("device ")]
    assert len(dev) >= 1
    for l in dev:
        assert l.split()[2:] == want
