import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu on the GPU box)")


@pytest.fixture(scope="session")
def cuda():
    """torch with a CUDA device; GPU tests fail loudly (never skip silently) when the library is missing."""
    import torch
    assert torch.cuda.is_available(), "a -m gpu test ran without a CUDA device"
    import infer_b200
    infer_b200.lib()  # raises if libfth_b200.so is not built
    return torch
