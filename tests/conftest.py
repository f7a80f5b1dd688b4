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
    # One OpenMP thread: the reference's cooperative multi-thread axis reduction (omp2 mode of
    # solid/include/solid/core/cpu/reduce_axis.h:456-640) mis-steps when a thread's share of a
    # multi-dimensional reduced range starts inside a row (ridx[0] is never reset, line 574), so
    # its results there depend on the thread count; the sequential path is the well-defined oracle.
    c.set_threads(1)
    return c
