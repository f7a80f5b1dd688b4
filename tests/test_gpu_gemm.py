"""Parity of the integer and boolean matrix product solid_gpu_gemm_<type> with the reference's Solid CPU
library (solid/src/core/cpu/template_blas.c): C = alpha * op(A) * op(B) + beta * C in the wrap-around
arithmetic of the element type (bool: and / or).  Bit-exact.  8- and 16-bit types use their full range (the
narrowing on every store makes wrap-around defined on the CPU too); 32- and 64-bit operands stay small enough
that no signed intermediate overflows there.
"""
import numpy as np
import pytest

import util
from solid_b200 import dtypes as dt

pytestmark = pytest.mark.gpu

SHAPES = [(1, 1, 1), (5, 7, 3), (33, 65, 40), (64, 32, 100), (31, 1, 257), (4, 6, 0), (0, 5, 3)]


def operands(dtype, rng, rows, cols, ld):
    """Column-major rows x cols matrix inside a buffer with leading dimension ld (elements)."""
    npdt = dt.NUMPY[dtype]
    n = ld * max(cols, 1)
    if dtype == "bool":
        vals = (rng.random(n) < 0.3).astype(np.uint8)
    elif dt.SIZE[dtype] <= 2:
        info = np.iinfo(npdt)
        vals = rng.integers(info.min, int(info.max) + 1, n).astype(npdt)
    else:
        vals = rng.integers(-50 if dtype.startswith("int") else 0, 50, n).astype(npdt)
    return vals


@pytest.mark.parametrize("dtype", dt.GROUPS["integer_bool"])
def test_gemm_matches_reference(dtype, gpu, cpu):
    dev = util.Device()
    rng = np.random.default_rng(900 + dt.INDEX[dtype])
    npdt = dt.NUMPY[dtype]
    scalars = [(1, 0), (1, 1), (0, 1), (0, 0)] if dtype == "bool" else [(1, 0), (3, 2), (0, 5), (0, 1), (2, 0)]
    if dtype.startswith("int"):
        scalars.append((-2, -1))
    for (m, n, k) in SHAPES:
        for ta in "NT":
            for tb in "nT":
                ra, ca = (m, k) if ta == "N" else (k, m)
                rb, cb = (k, n) if tb in "nN" else (n, k)
                lda, ldb, ldc = ra + 3, rb + 1, m + 2
                A = operands(dtype, rng, ra, ca, lda); B = operands(dtype, rng, rb, cb, ldb)
                C0 = operands(dtype, rng, m, n, ldc)
                for case, (alpha, beta) in enumerate(scalars):
                    al = np.array([alpha]).astype(npdt); be = np.array([beta]).astype(npdt)
                    want = C0.copy()
                    cpu.gemm(dtype, ta, tb, m, n, k, al.ctypes.data, A.ctypes.data, lda, B.ctypes.data, ldb,
                             be.ctypes.data, want.ctypes.data, ldc)
                    dA, dB, dC = dev.upload(A.view(np.uint8)), dev.upload(B.view(np.uint8)), dev.upload(C0.view(np.uint8))
                    if case % 2 == 0:         # scalars in host memory
                        gpu.gemm(dtype, ta, tb, m, n, k, al.ctypes.data, dA.data_ptr(), lda, dB.data_ptr(), ldb,
                                 be.ctypes.data, dC.data_ptr(), ldc, True, dev.stream)
                    else:                     # scalars in device memory
                        dal, dbe = dev.upload(al.view(np.uint8)), dev.upload(be.view(np.uint8))
                        gpu.gemm(dtype, ta, tb, m, n, k, dal.data_ptr(), dA.data_ptr(), lda, dB.data_ptr(), ldb,
                                 dbe.data_ptr(), dC.data_ptr(), ldc, False, dev.stream)
                    got = dev.download(dC)[: C0.nbytes].view(npdt)
                    assert np.array_equal(got, want), (dtype, (m, n, k), ta, tb, alpha, beta,
                                                       np.nonzero(got != want)[0][:5])
    # absent scalars: alpha = 1, beta = 0
    m, n, k = 17, 9, 12
    A = operands(dtype, rng, m, k, m); B = operands(dtype, rng, k, n, k); C0 = operands(dtype, rng, m, n, m)
    want = C0.copy()
    cpu.gemm(dtype, "N", "N", m, n, k, None, A.ctypes.data, m, B.ctypes.data, k, None, want.ctypes.data, m)
    dA, dB, dC = dev.upload(A.view(np.uint8)), dev.upload(B.view(np.uint8)), dev.upload(C0.view(np.uint8))
    gpu.gemm(dtype, "N", "N", m, n, k, None, dA.data_ptr(), m, dB.data_ptr(), k, None, dC.data_ptr(), m, True, dev.stream)
    assert np.array_equal(dev.download(dC)[: C0.nbytes].view(npdt), want), (dtype, "absent scalars")


def test_gemm_rejects_unknown_modes(gpu):
    from solid_b200._lib import SolidError
    dev = util.Device()
    d = dev.empty(256)
    with pytest.raises(SolidError, match="Invalid mode"):
        gpu.gemm("int32", "X", "N", 2, 2, 2, None, d.data_ptr(), 2, d.data_ptr(), 2, None, d.data_ptr(), 2, True, dev.stream)
