import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def native():
    """Builds (if needed) and loads the native library."""
    from cutt_b200 import build as _build
    _build.build()
    import cutt_b200
    cutt_b200.lib()
    return cutt_b200


@pytest.fixture(scope="session")
def oracle_mod():
    import oracle
    oracle.load()
    return oracle
