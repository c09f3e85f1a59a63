#!/usr/bin/env python3
"""Produce tests/golden/reference_cases.json from the reference's own unit tests.

Runs only where the reference checkout is present (it is read, never copied):
each listed *_test.cc is compiled, unmodified, against this repository's
tim::vx headers, a small GoogleTest stand-in (tests/golden/shim) and the
oracle-backed libraries (oracle/_build), then executed.  The oracle backend
writes one JSON case per graph run: tensors, nodes, inputs, its own outputs and
the vector the test compared against.  Those cases are packed (arrays as
base64(zlib(raw bytes))) into reference_cases.json, and a one-line-per-test
verdict of "reference test vs oracle" goes to reference_report.txt.

usage: python tests/golden/make_goldens.py --reference <TIM-VX source tree>
"""
import argparse
import base64
import glob
import json
import os
import subprocess
import sys
import tempfile
import zlib

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))

TEST_FILES = [
    "src/tim/vx/ops/conv2d_test.cc",
    "src/tim/vx/ops/depthwiseConv_test.cc",
    "src/tim/vx/ops/avg_pool_test.cc",
    "src/tim/vx/ops/max_pool_test.cc",
    "src/tim/vx/ops/fullyconnected_test.cc",
    "src/tim/vx/ops/softmax_test.cc",
    "src/tim/vx/ops/transpose_test.cc",
    "src/tim/vx/ops/groupedconv2d_test.cc",
    "src/tim/vx/ops/addn_test.cc",
    "src/tim/vx/ops/simple_operations_test.cc",
    "src/tim/vx/ops/reshape_test.cc",
    "src/tim/transform/layout_inference_test.cc",
    "src/tim/transform/average_pool_layout_infer_test.cc",
    "src/tim/vx/graph_test.cc",
]


def pack(hexstr):
    if hexstr is None:
        return None
    raw = bytes.fromhex(hexstr)
    return base64.b64encode(zlib.compress(raw, 9)).decode("ascii")


NP_DTYPE = {1: "i1", 2: "u1", 5: "<i4", 9: "<f4"}


def max_diff(case):
    """Largest |oracle output - expected| over the expectations of one case (before packing)."""
    import numpy as np
    worst = 0.0
    for e in case["expect"]:
        t = case["tensors"][e["tensor"]]
        if t["data"] is None:
            continue
        got = np.frombuffer(zlib.decompress(base64.b64decode(t["data"])), NP_DTYPE[t["dtype"]]).astype("f8")
        want = np.frombuffer(zlib.decompress(base64.b64decode(e["data"])), NP_DTYPE[e["dtype"]]).astype("f8")
        if got.shape == want.shape and got.size:
            worst = max(worst, float(np.abs(got - want).max()))
    return worst


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="root of a TIM-VX v1.2.22 source tree")
    args = ap.parse_args()
    ref = args.reference
    subprocess.check_call(["make", "-C", os.path.join(ROOT, "oracle")], stdout=subprocess.DEVNULL)
    build = os.path.join(ROOT, "oracle", "_build")
    shim = os.path.join(HERE, "shim")
    cases, report = [], []
    with tempfile.TemporaryDirectory() as tmp:
        for rel in TEST_FILES:
            src = os.path.join(ref, rel)
            exe = os.path.join(tmp, os.path.basename(rel) + ".exe")
            cap = os.path.join(tmp, os.path.basename(rel) + ".cap")
            os.makedirs(cap)
            cmd = ["/usr/bin/g++", "-std=c++17", "-O1", "-w",
                   "-DREFERENCE_TEST_UTILS_H=\"%s\"" % os.path.join(ref, "src/tim/vx/test_utils.h"),
                   "-I" + shim, "-I" + os.path.join(shim, "stubs"), "-I" + os.path.join(ROOT, "include"), "-I" + ref,
                   src, os.path.join(shim, "gtest_main.cc"),
                   "-L" + build, "-ltim-vx-oracle", "-lb2vx_oracle", "-Wl,-rpath," + build, "-o", exe]
            cc = subprocess.run(cmd, capture_output=True, text=True)
            if cc.returncode != 0:
                report.append("COMPILE_ERROR %s\n%s" % (rel, cc.stderr[-2000:]))
                continue
            env = dict(os.environ, B2VX_CAPTURE_DIR=cap, VSI_NN_LOG_LEVEL="0")
            run = subprocess.run([exe], capture_output=True, text=True, env=env)
            verdicts = [(line.split()[0], " ".join(line.split()[1:])) for line in run.stdout.splitlines()]
            diffs = {}
            for path in sorted(glob.glob(os.path.join(cap, "*.json"))):
                c = json.load(open(path))
                c["source"] = rel
                for t in c["tensors"]:
                    t["data"] = pack(t["data"])
                for e in c["expect"]:
                    e["data"] = pack(e["data"])
                if c["expect"]:
                    cases.append(c)
                    diffs[c["name"]] = max(diffs.get(c["name"], 0.0), max_diff(c))
            for verdict, name in verdicts:
                note = ""
                if name in diffs:
                    note = "  (max |oracle - expected| = %.3g)" % diffs[name]
                elif verdict in ("FAIL", "CRASH"):
                    note = "  (op or dtype outside the quantized CNN path: float16, int16 DFP, Pool1d, declared-only ops)"
                report.append("%-8s %s :: %s%s" % (verdict, rel, name, note))
    with open(os.path.join(HERE, "reference_cases.json"), "w") as f:
        json.dump({"format": "b64(zlib(raw little-endian bytes)), dims fastest-first", "cases": cases}, f,
                  separators=(",", ":"))
    with open(os.path.join(HERE, "reference_report.txt"), "w") as f:
        f.write("\n".join(report) + "\n")
    print("\n".join(report))
    print("%d cases written" % len(cases))
    return 0


if __name__ == "__main__":
    sys.exit(main())
