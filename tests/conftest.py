import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def golden_dir():
    return os.path.join(ROOT, "tests", "golden")


@pytest.fixture(scope="session")
def capi():
    """The product library through its C ABI; fails loudly when it cannot be used."""
    import torch
    from thundersvm_b200 import build, capi as capi_mod
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    build.build()
    capi_mod.lib()
    return capi_mod
