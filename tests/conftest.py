"""Shared fixtures. Tests marked `gpu` need a B200 and call the CUDA library through its C ABI;
everything else runs on CPU (oracle against golden vectors, host logic, exported symbols)."""
import importlib.util
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def load_hb200():
    """Imports the package directory (its name is not an identifier) as module `hb200`."""
    if "hb200" in sys.modules:
        return sys.modules["hb200"]
    path = os.path.join(ROOT, "herbert-metal-bf16_b200", "__init__.py")
    spec = importlib.util.spec_from_file_location("hb200", path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules["hb200"] = mod
    spec.loader.exec_module(mod)
    return mod


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200; runs the CUDA kernels through the C ABI")


@pytest.fixture(scope="session")
def hb200():
    return load_hb200()


@pytest.fixture(scope="session")
def oracle():
    from oracle_lib import Oracle

    return Oracle()


@pytest.fixture(scope="session")
def ctx(hb200):
    """One context for the whole GPU session. A missing library or device is an error, not a skip:
    the GPU tests must never pass on anything but the CUDA path."""
    c = hb200.Context(0)
    yield c
    c.close()
