import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def pkg():
    """The ctypes binding of the CUDA library (built on demand when nvcc is present)."""
    import __graft_entry__ as ge
    ge._load_file("b200attn_build", os.path.join(ge.PKG_DIR, "build.py")).build()
    return ge.load_package()


@pytest.fixture(scope="session")
def cuda(pkg):
    import torch
    if not torch.cuda.is_available():
        pytest.fail("this test is marked gpu and needs a CUDA device; there is no CPU fallback")
    return torch.device("cuda:0")
