import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def built():
    """The native libraries, built in-tree if they are stale or missing."""
    from turbotransformers_b200 import build
    return build.build_all()


@pytest.fixture(scope="session")
def ctx(built):
    """A C-ABI context on cuda:0 running on torch's current stream."""
    import torch
    from turbotransformers_b200 import _capi
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    c = _capi.Context(0)
    yield c
    torch.cuda.synchronize()
    c.close()
