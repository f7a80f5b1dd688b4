import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "ocean-tensor-package_b200"))
sys.path.insert(0, str(ROOT / "tests"))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def gpu():
    """The C-ABI library bound with ctypes, on cuda:0.  No fallback of any kind."""
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from solid_b200 import _lib
    lib = _lib.get()
    torch.cuda.set_device(0)
    lib.initialize()
    return lib


@pytest.fixture(scope="session")
def cpu():
    """The reference's Solid CPU library (the oracle)."""
    from oracle import ref
    if not ref.available():
        pytest.skip("oracle/_ref/libsolid_core_cpu.so not built")
    c = ref.get()
    return c
