import importlib
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu on the GPU box)")


@pytest.fixture(scope="session")
def t0():
    """The host-side binding package (directory name has a hyphen)."""
    mod = importlib.import_module("rust-gpu_b200")
    if not os.path.exists(mod.LIB_PATH):
        mod.build()
    mod.lib()
    return mod


@pytest.fixture(scope="session")
def oracle():
    import oracle as _oracle
    _oracle.build()
    _oracle.lib()
    return _oracle


@pytest.fixture(scope="session")
def golden_dir():
    return os.path.join(ROOT, "tests", "golden")


@pytest.fixture()
def rt(t0):
    """A GpuRuntime; like the reference's shared test runtime it is rebuilt when poisoned
    (src/t0/tile_ir.rs:4980-5004)."""
    r = _shared_runtime(t0)
    yield r


_RT = {}


def _shared_runtime(t0):
    r = _RT.get("rt")
    if r is None or r.is_poisoned():
        r = t0.GpuRuntime(0)
        _RT["rt"] = r
    return r
