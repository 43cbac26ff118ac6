import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def oracle():
    from tests.oracle_lib import Oracle
    return Oracle()


@pytest.fixture(scope="session")
def cuda_lib():
    """The product library; there is no fallback, so a GPU test without it fails."""
    import torch
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    from adop_b200 import capi
    return capi.load_library()
