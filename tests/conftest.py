import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (sm_100); run with -m gpu")


@pytest.fixture(scope="session")
def oracle():
    from oracle import oracle as mod
    mod.build()
    return mod


@pytest.fixture(scope="session")
def cuda_device():
    import torch
    if not torch.cuda.is_available():
        pytest.fail("a test marked gpu ran without a CUDA device; there is no CPU fallback")
    torch.cuda.set_device(0)
    return torch.device("cuda:0")
