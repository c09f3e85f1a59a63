"""pytest configuration: the `gpu` marker, import path, and library fixtures."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "tim-vx_b200"))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def _ensure(path, make_dir):
    if not os.path.exists(path):
        subprocess.check_call(["make", "-C", make_dir], stdout=subprocess.DEVNULL)
    return path


@pytest.fixture(scope="session")
def oracle_lib():
    import oracle_paths
    _ensure(oracle_paths.ORACLE_LIB, os.path.join(ROOT, "oracle"))
    return oracle_paths.load(oracle_paths.ORACLE_LIB)


@pytest.fixture(scope="session")
def product_lib():
    """The CUDA library.  Missing library = hard failure, never a fallback."""
    import pyb2vx
    assert os.path.exists(pyb2vx.PRODUCT_LIB), "libb2vx.so is not built: run python -c 'import __graft_entry__ as g; g.build()'"
    return pyb2vx.load(pyb2vx.PRODUCT_LIB)


@pytest.fixture(scope="session")
def reference_cases():
    with open(os.path.join(ROOT, "tests", "golden", "reference_cases.json")) as f:
        return json.load(f)["cases"]
