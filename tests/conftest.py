import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def lib():
    """The compiled C-ABI library (built on demand; building needs nvcc, not a GPU)."""
    from tracea_b200 import build, ffi
    build.build()
    return ffi.load()
