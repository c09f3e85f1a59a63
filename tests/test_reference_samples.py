"""The reference's own sample programs, compiled unmodified against this repository's headers.

`make -C oracle ref-samples REFERENCE=<reference tree>` compiles samples/lenet, samples/lenet_multi_device,
samples/multi_thread_test, samples/platform_sample and samples/benchmark_test from the reference tree, each
once on the oracle libraries (<name>.oracle) and once on the product libraries (<name>.gpu).  The sources
never enter this repository; only the binaries exist, beside the oracle, and they travel with the built
libraries.  The tests are skipped where the binaries were not built.

The same target links tests/cpp/exported_graphs.cc with the reference's three generated graph sources
(samples/multi_device/vx_lenet.cc, vx_mobilenet.cc, vx_resnet50.cc) and writes their data files
(oracle/make_export_blobs.py).

What a sample prints (LeNet's top-5 classes with their probabilities for the digit image the sample
carries, the sums of the platform sample) must be the same text on the oracle, on the GPU, and in the
committed expectation under tests/golden/reference_samples/.
"""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BIN = os.path.join(ROOT, "oracle", "_ref")
GOLDEN = os.path.join(ROOT, "tests", "golden", "reference_samples")

# name, command-line arguments, golden file
SAMPLES = [
    ("lenet_asymu8", [], "lenet_asymu8.txt"),
    ("lenet_multi_device", [], "lenet_multi_device.txt"),
    ("multi_thread_test", [], "multi_thread_test.txt"),
    ("platform_sample", [], "platform_sample.txt"),
    ("benchmark_test", ["56", "56", "64", "3", "3", "64", "0"], "benchmark_test_conv.txt"),
    ("benchmark_test", ["56", "56", "32", "3", "3", "32", "1"], "benchmark_test_depthwise.txt"),
]
IDS = [s[2][:-4] for s in SAMPLES]


def normalise(name, text):
    """Lines that may legitimately differ between machines are dropped: the device census of the platform
    sample.  The two threads of multi_thread_test write to std::cout without a lock, so their output
    interleaves piece by piece; what is invariant is the multiset of printed characters, which still pins
    every digit of both threads' probabilities."""
    if name == "multi_thread_test":
        return ["".join(sorted("".join(text.split())))]
    lines = [l.rstrip() for l in text.splitlines() if l.strip()]
    return [l for l in lines if not l.startswith("NPU device")]


def run(name, args, flavour):
    exe = os.path.join(BIN, "%s.%s" % (name, flavour))
    if not os.path.exists(exe):
        pytest.skip("reference samples were not built (make -C oracle ref-samples REFERENCE=<tree>)")
    r = subprocess.run([exe] + args, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, "%s exited %d\n%s\n%s" % (exe, r.returncode, r.stdout[-1500:], r.stderr[-1500:])
    return normalise(name, r.stdout)


def golden(name, fname):
    with open(os.path.join(GOLDEN, fname)) as f:
        return normalise(name, f.read())


@pytest.mark.parametrize("name,args,fname", SAMPLES, ids=IDS)
def test_reference_sample_on_oracle(name, args, fname):
    assert run(name, args, "oracle") == golden(name, fname)


@pytest.mark.gpu
@pytest.mark.parametrize("name,args,fname", SAMPLES, ids=IDS)
def test_reference_sample_on_gpu(name, args, fname):
    got = run(name, args, "gpu")
    assert got == golden(name, fname)
    assert got == run(name, args, "oracle")


EXPORT_DATA = os.path.join(BIN, "export_data")


def run_exported(flavour):
    exe = os.path.join(BIN, "exported_graphs.%s" % flavour)
    if not os.path.exists(exe) or not os.path.isdir(EXPORT_DATA):
        pytest.skip("the exported graphs were not built (make -C oracle ref-samples REFERENCE=<tree>)")
    r = subprocess.run([exe, EXPORT_DATA], capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, "%s exited %d\n%s\n%s" % (exe, r.returncode, r.stdout[-1500:], r.stderr[-1500:])
    lines = [l.strip() for l in r.stdout.splitlines() if l.startswith(("lenet:", "mobilenet:", "resnet50:", "ok "))]
    assert lines[-1] == "ok exported graphs"
    return lines


def test_exported_graphs_on_oracle():
    """The reference's generated graph sources (samples/multi_device/vx_lenet.cc, vx_mobilenet.cc, vx_resnet50.cc),
    unmodified: LeNet with its real coefficient file must name the class the reference's LeNet sample names for the
    same digit; the other two run on seeded stand-in coefficients and must give a non-degenerate distribution."""
    lines = run_exported("oracle")
    with open(os.path.join(GOLDEN, "lenet_asymu8.txt")) as f:
        top = [l for l in f.read().splitlines() if l.strip() and l.split(":")[0].strip().isdigit()]
    best_class = int(top[0].split(":")[0])
    assert ("top-1 class %d," % best_class) in lines[0], (lines[0], top[0])
    for l in lines[1:3]:
        assert float(l.rsplit(" ", 1)[1]) > 0.01, l     # far from the uniform 1/1000


@pytest.mark.gpu
def test_exported_graphs_on_gpu_match_oracle():
    """Same programs on the CUDA libraries: every network must name the oracle's best class with the oracle's
    probability within 1e-5 (the outputs are float32 softmax values; device expf against libm is this repository's
    one stated float tolerance, so the byte hash the driver prints is informative only)."""
    want, got = run_exported("oracle"), run_exported("gpu")
    assert len(want) == len(got) == 4
    for w, g in zip(want[:3], got[:3]):
        wf, gf = w.split(), g.split()
        assert wf[0] == gf[0] and wf[1] == gf[1]                      # name, output count
        assert wf[wf.index("class") + 1] == gf[gf.index("class") + 1], (w, g)
        assert abs(float(wf[-1]) - float(gf[-1])) <= 1e-5, (w, g)


def test_product_sample_binary_refuses_to_run_without_a_gpu(product_lib):
    """No CPU fallback behind the reference's program either: without a CUDA device it reports the failure."""
    if product_lib.b2vx_device_count() > 0:
        pytest.skip("a GPU is present")
    exe = os.path.join(BIN, "lenet_asymu8.gpu")
    if not os.path.exists(exe):
        pytest.skip("reference samples were not built")
    r = subprocess.run([exe], capture_output=True, text=True, timeout=120)
    assert "Top5" not in r.stdout
    assert "no CUDA device" in r.stderr
