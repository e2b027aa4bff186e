"""Shared test plumbing: the `gpu` marker, the package loaded by path, the oracle doors."""
import importlib.util
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG_DIR = os.path.join(ROOT, "tetris-artifact-evalution_b200")
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def load_package():
    """Import the engine package (its directory name has a hyphen) as `tetris_b200`."""
    if "tetris_b200" in sys.modules:
        return sys.modules["tetris_b200"]
    spec = importlib.util.spec_from_file_location(
        "tetris_b200", os.path.join(PKG_DIR, "__init__.py"), submodule_search_locations=[PKG_DIR])
    mod = importlib.util.module_from_spec(spec)
    sys.modules["tetris_b200"] = mod
    spec.loader.exec_module(mod)
    return mod


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def tb():
    return load_package()


@pytest.fixture(scope="session")
def workloads(tb):
    import importlib
    return importlib.import_module("tetris_b200.workloads")


@pytest.fixture(scope="session")
def oracle():
    from oracle import oracle as orc
    orc.port()
    return orc


@pytest.fixture(scope="session")
def torch_cuda():
    import torch
    if not torch.cuda.is_available():
        pytest.fail("a test marked gpu ran without a CUDA device")
    torch.cuda.set_device(0)
    return torch
