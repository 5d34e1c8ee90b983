"""pytest configuration: registers the `gpu` marker, puts the package on sys.path and builds the
native library on first use if it is not there yet."""
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "amd-kernels_b200")
for p in (ROOT, PKG):
    if p not in sys.path:
        sys.path.insert(0, p)

LIB = os.path.join(PKG, "kernels", "libhkb200.so")
GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")
    if not os.path.exists(LIB):
        import importlib.util
        spec = importlib.util.spec_from_file_location("hkb_build", os.path.join(PKG, "build.py"))
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        mod.build()


def pytest_collection_modifyitems(config, items):
    import torch
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def hk():
    import hipkittens
    return hipkittens


@pytest.fixture(scope="session")
def golden_dir():
    return GOLDEN
