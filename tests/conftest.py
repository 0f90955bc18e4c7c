import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (sm_100) GPU and the built session library")


@pytest.fixture(scope="session")
def cuda_lib():
    """The session library, loaded or the test fails: there is no CPU fallback."""
    from altius_b200 import session
    lib = session.load_library()
    n = lib.altius_cuda_device_count()
    assert n > 0, "no CUDA device visible to the session library"
    return lib
