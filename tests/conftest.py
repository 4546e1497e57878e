import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def sgemm():
    """The product package with its compiled library; built on demand where nvcc exists."""
    import rocm_sgemm_b200 as r
    if not os.path.exists(r.LIB_PATH):
        from rocm_sgemm_b200 import build
        build.build_library()
    r.lib()
    return r


@pytest.fixture(scope="session")
def orc():
    import oracle
    oracle.lib()
    return oracle
