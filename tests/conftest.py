import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import __graft_entry__ as entry  # noqa: E402


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu on the GPU box)")


@pytest.fixture(scope="session")
def pkg():
    return entry.load_package()


@pytest.fixture(scope="session")
def oracle():
    o = entry.load_oracle()
    o.build()
    return o


@pytest.fixture(scope="session")
def cuda(pkg):
    """torch with a CUDA device and the built library; GPU tests fail (not
    skip) when the extension is missing."""
    import torch
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    pkg.lib.load()
    torch.cuda.set_device(0)
    return torch
