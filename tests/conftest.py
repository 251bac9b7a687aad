import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200, sm_100a)")


@pytest.fixture(scope="session")
def kat():
    return np.load(os.path.join(ROOT, "tests", "golden", "kat.npz"))


@pytest.fixture(scope="session")
def oracle():
    from oracle import oracle as O
    O.build()
    return O


@pytest.fixture(scope="session")
def ctx():
    """One context for the whole GPU session (one context per host thread per GPU)."""
    import rusty_b200
    c = rusty_b200.CudaContext(0)
    yield c
    c.destroy()


@pytest.fixture(scope="session")
def engine(ctx):
    import rusty_b200
    return rusty_b200.ComputeEngine(ctx)


@pytest.fixture(autouse=True)
def _guard_zones_intact(request):
    """After every GPU test that used the shared context: the guard zones between the kernels' scratch regions
    must be untouched (the tests' stand-in for a memory checker, which cannot be run on these GPUs)."""
    yield
    if request.node.get_closest_marker("gpu") is not None and "ctx" in request.fixturenames:
        request.getfixturevalue("ctx").self_check()
