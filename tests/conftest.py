import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200; run with -m gpu")


@pytest.fixture(scope="session")
def golden():
    import numpy as np
    return np.load(os.path.join(ROOT, "tests", "golden", "golden.npz"))


@pytest.fixture(scope="session")
def lib():
    """The built C-ABI library (compiled on first use if the .so is stale)."""
    from cute_rs_b200 import _lib, build
    build.build()
    return _lib


@pytest.fixture(scope="session")
def gpu(lib):
    """Device 0 initialised for the library; fails loudly without one."""
    import torch
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    lib.init(0)
    return torch.device("cuda:0")
