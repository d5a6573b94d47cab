import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import __graft_entry__ as entry  # noqa: E402


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")
    config.addinivalue_line("markers", "strict_default: host-pointer test that keeps the library's default fold order")


@pytest.fixture(scope="session")
def O():
    """The CPU oracle (the checker)."""
    return entry.load_oracle()


@pytest.fixture(scope="session")
def pkg():
    """The provider package; GPU tests call the C ABI through it."""
    return entry.load_package()


@pytest.fixture(scope="session")
def cuda(pkg):
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    if not os.path.exists(pkg.LIB_PATH):
        pytest.fail("libtcrv_cuda.so is not built; GPU tests have no fallback to run on")
    pkg.lib()
    torch.cuda.set_device(0)
    return torch
