import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

# every launch made by the tests reads the device status word back
os.environ.setdefault("XATTN_B200_SYNC_CHECK", "1")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (sm_100) GPU and the built libxattn_b200.so")


@pytest.fixture(scope="session")
def cuda_device():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("CUDA unavailable")
    if torch.cuda.get_device_capability()[0] != 10:
        pytest.skip("sm_100 required")
    from xattn_b200 import _lib
    _lib.load()  # a missing library is an error on a GPU box, not a skip
    return torch.device("cuda")
