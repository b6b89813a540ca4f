"""Shared fixtures. GPU tests are marked `gpu`; everything else runs on CPU."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

KERNEL_CACHE = os.path.join(ROOT, ".kernel_cache")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu)")


@pytest.fixture(scope="session")
def built():
    """Builds the product library and the oracle once per session."""
    import __graft_entry__
    __graft_entry__.build()
    from libgpuarray_b200 import api
    return api


@pytest.fixture(scope="session")
def api(built):
    return built


@pytest.fixture(scope="session")
def oracle(built):
    from oracle import oracle as O
    O.lib()
    return O


@pytest.fixture(scope="session")
def ctx(api):
    c = api.Context(0, kernel_cache=KERNEL_CACHE)
    yield c
    c.close()


@pytest.fixture()
def rng():
    return np.random.default_rng(12345)
