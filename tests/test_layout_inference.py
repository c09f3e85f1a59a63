"""tim::transform::LayoutInference (tests/cpp/layout_inference.cc): the reference's two convolution cases
(src/tim/transform/layout_inference_test.cc:9-121), and a quantized NHWC network whose inferred graph must
give the same bytes as the same network written natively in WHCN, with no Transpose beyond the one at the
input and the one in front of the FullyConnected.  The program runs on the oracle build (CPU test) and on
the CUDA build (GPU test), which must print the same logits."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC = os.path.join(ROOT, "tests", "cpp", "layout_inference.cc")


def build(tmp_path, libdir, libs, name):
    exe = str(tmp_path / name)
    subprocess.check_call(["/usr/bin/g++", "-std=c++17", "-O1", "-Wall", "-Wextra", "-Werror", "-I" + os.path.join(ROOT, "include"), SRC,
                           "-L" + libdir] + ["-l" + l for l in libs] + ["-Wl,-rpath," + libdir, "-o", exe])
    return exe


def run(exe):
    out = subprocess.run([exe], capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, "exit %d\n%s%s" % (out.returncode, out.stdout, out.stderr)
    lines = out.stdout.strip().splitlines()
    assert lines[-1] == "ok layout inference"
    return [l for l in lines if l.startswith("logits ")][0]


def test_layout_inference_on_the_oracle(tmp_path, oracle_lib):
    logits = run(build(tmp_path, os.path.join(ROOT, "oracle", "_build"), ["tim-vx-oracle", "b2vx_oracle"], "layout_oracle")).split()[1:]
    assert len(set(logits)) > 4


@pytest.mark.gpu
def test_layout_inference_on_gpu_matches_oracle(tmp_path, oracle_lib, product_lib):
    want = run(build(tmp_path, os.path.join(ROOT, "oracle", "_build"), ["tim-vx-oracle", "b2vx_oracle"], "layout_oracle"))
    got = run(build(tmp_path, os.path.join(ROOT, "tim-vx_b200", "csrc"), ["tim-vx", "b2vx"], "layout_gpu"))
    assert got == want
