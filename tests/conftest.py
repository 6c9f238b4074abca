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
    """Builds (if needed) and loads the native library.

    Most test tensors are small enough for the planner to hand them to the element-per-thread
    kernel; that candidate is switched off here so that the tiled kernels keep serving the shapes
    these tests were written for.  The tests of the small-tensor path switch it back on."""
    from cutt_b200 import build as _build
    _build.build()
    import cutt_b200
    cutt_b200.lib()
    os.environ["CUTT_NO_NAIVE_CANDIDATE"] = "1"
    return cutt_b200


@pytest.fixture(scope="session")
def oracle_mod():
    import oracle
    oracle.load()
    return oracle
