import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 and the built libvknn_cuda.so")


@pytest.fixture(scope="session")
def ctx():
    """One libvknn_cuda context on cuda:0. No fallback: a missing library or device is a test error."""
    import torch
    import vknn_b200
    assert torch.cuda.is_available(), "gpu tests need a CUDA device"
    torch.cuda.set_device(0)
    c = vknn_b200.Context(0)
    yield c
    c.sync()
    c.close()
