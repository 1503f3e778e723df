"""Shared pytest setup: import paths, the ``gpu`` marker and an in-tree build of the C-ABI library."""

import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
for p in (ROOT, ROOT / "pith-train_b200"):
    if str(p) not in sys.path:
        sys.path.insert(0, str(p))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def built_library():
    """Path of libpith_b200.so, compiled with nvcc if it is missing or stale."""
    from pithtrain_b200 import build
    return build.build_library()


@pytest.fixture(scope="session")
def cuda_device(built_library):
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda", 0)
