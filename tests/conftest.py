import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA GPU (the kernels target B200, sm_100a)")


@pytest.fixture(scope="session")
def golden_dir():
    return os.path.join(ROOT, "tests", "golden")


@pytest.fixture(scope="session")
def cuda_lib():
    """The C-ABI library, loaded on a machine with a GPU; GPU tests fail (not skip) if it is missing."""
    import torch

    assert torch.cuda.is_available(), "GPU test selected on a machine without CUDA"
    from lightning_attention_b200 import _lib

    return _lib.lib()
