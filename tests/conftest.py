"""pytest configuration: the `gpu` marker, import paths, and the two libraries' bindings.

`-m "not gpu"` runs on a machine without a GPU: the oracle against the golden vectors and the reference's own host
code (where it was built), the product's host logic, and the C-ABI symbol check.  `-m gpu` is the parity suite proper
and calls the CUDA path through the C ABI.
"""
import importlib
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (sm_100a) GPU; run with -m gpu")


def _product():
    mod = sys.modules.get("ling_engine_b200")
    if mod is None:
        mod = importlib.import_module("ling-engine_b200")
        sys.modules["ling_engine_b200"] = mod
    return mod


@pytest.fixture(scope="session")
def lb():
    """The product binding (ling-engine_b200); building the library first if it is missing."""
    mod = _product()
    if not os.path.exists(mod.LIB_PATH):
        importlib.import_module("ling-engine_b200.build").build()
    mod.lib()
    return mod


@pytest.fixture(scope="session")
def lo():
    """The oracle binding (test infrastructure)."""
    from oracle import lo as m
    m.lo()
    return m


@pytest.fixture(scope="session")
def gpu(lb):
    """Skips unless a GPU is present; GPU tests must also carry the `gpu` marker."""
    if lb.lib().ling_b200_device_count() < 1:
        pytest.skip("no CUDA device")
    return 0
