"""Shared fixtures.  Tests marked `gpu` need a B200 and call the CUDA path through the C ABI; the
rest run on CPU (oracle pinning, host logic, library loading)."""
import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); runs the CUDA kernels")


@pytest.fixture(scope="session")
def built():
    """The in-tree libraries, built on demand (nvcc cross-compiles without a GPU)."""
    from mantle_b200 import build as b
    b.build_all()
    return b


@pytest.fixture(scope="session")
def oracle_mod():
    import oracle
    oracle.build()
    return oracle


@pytest.fixture(scope="session")
def ctx(built):
    import mantle_b200 as mb
    c = mb.Context(0)
    yield c
    c.close()
