import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the GPU box)")


@pytest.fixture(scope="session")
def oracle():
    from oracle import eigenmat_oracle
    return eigenmat_oracle


@pytest.fixture(scope="session")
def cm():
    """The CUDA backend.  No skip and no fallback: a missing device or library is a failure."""
    from deepnet_b200 import b200mat
    b200mat.cublas_init()
    return b200mat
