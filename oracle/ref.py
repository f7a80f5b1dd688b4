"""ctypes access to the reference's Solid CPU library (oracle/_ref/libsolid_core_cpu.so).

TEST INFRASTRUCTURE: the checker the CUDA path is compared with, and the timed
CPU baseline.  The library is the unmodified reference code, built by
oracle/build_ref.py; its entry points are declared in the reference's
solid/src/core/cpu/solid_core_cpu.src (elementwise :106-255, copy :27-52,
global reductions :263-332, axis reductions :341-413).  CPU signatures are the
GPU ones without stream and scratch buffer.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "_ref" / "libsolid_core_cpu.so"


def available() -> bool:
    return LIB_PATH.exists()


def _sizes(seq):
    return (C.c_size_t * max(len(seq), 1))(*seq)


def _strides(seq):
    return (C.c_ssize_t * max(len(seq), 1))(*seq)


class Scalar(C.Structure):
    """solid_scalar by value: first eightbyte INTEGER class, second SSE (see the x86-64 ABI);
    ctypes cannot pass the union itself by value."""
    _fields_ = [("lo", C.c_uint64), ("hi", C.c_double)]


def _scalar(raw: bytes) -> Scalar:
    s = Scalar()
    C.memmove(C.addressof(s), raw, min(len(raw), 16))
    return s


class CDouble(C.Structure):
    _fields_ = [("real", C.c_double), ("imag", C.c_double)]


class SolidCPU:
    def __init__(self, path=LIB_PATH):
        if not Path(path).exists():
            raise ImportError("%s is missing: run oracle/build_ref.py where the reference checkout is present" % path)
        self.dll = C.CDLL(str(path))

    def errmsg(self):
        return (C.c_char_p.in_dll(self.dll, "solid_errmsg").value or b"").decode(errors="replace")

    def _check(self, st, what):
        if st != 0:
            raise RuntimeError("%s: %s" % (what, self.errmsg()))

    def fn(self, name):
        f = getattr(self.dll, name)
        f.restype = C.c_int
        return f

    def has(self, name):
        return hasattr(self.dll, name)

    def set_threads(self, n: int):
        """OpenMP threads used by the reference (its float reduction order depends on it)."""
        import os
        os.environ["OMP_NUM_THREADS"] = str(n)
        try:
            C.CDLL("libgomp.so.1").omp_set_num_threads(C.c_int(n))
        except OSError:
            pass

    def fill(self, name, dtype, size, strides, ptr, value: bytes):
        self._check(self.fn("solid_cpu_%s_%s" % (name, dtype))(
            C.c_int(len(size)), _sizes(size), _strides(strides), C.c_void_p(ptr), _scalar(value)), name)

    def masked_fill(self, dtype, size, strides1, ptr1, strides2, ptr2, value: bytes):
        self._check(self.fn("solid_cpu_masked_fill_%s" % dtype)(
            C.c_int(len(size)), _sizes(size), _strides(strides1), C.c_void_p(ptr1), _strides(strides2),
            C.c_void_p(ptr2), _scalar(value)), "masked_fill")

    def unary(self, name, dtype, size, strides1, ptr1, strides2, ptr2):
        self._check(self.fn("solid_cpu_%s_%s" % (name, dtype))(
            C.c_int(len(size)), _sizes(size), _strides(strides1), C.c_void_p(ptr1),
            _strides(strides2), C.c_void_p(ptr2)), name)

    def binary(self, name, dtype, size, strides1, ptr1, strides2, ptr2, strides3, ptr3):
        self._check(self.fn("solid_cpu_%s_%s" % (name, dtype))(
            C.c_int(len(size)), _sizes(size), _strides(strides1), C.c_void_p(ptr1),
            _strides(strides2), C.c_void_p(ptr2), _strides(strides3), C.c_void_p(ptr3)), name)

    def steps(self, kind, dtype, size, strides, ptr, offset, step):
        """solid_cpu_steps_<kind>_<dtype> (solid/src/core/cpu/template_steps.c); kind 'int64', 'double', 'cdouble'."""
        f = self.fn("solid_cpu_steps_%s_%s" % (kind, dtype))
        if kind == "int64":
            args = (C.c_int64(int(offset)), C.c_int64(int(step)))
        elif kind == "double":
            args = (C.c_double(float(offset)), C.c_double(float(step)))
        else:
            args = (CDouble(complex(offset).real, complex(offset).imag), CDouble(complex(step).real, complex(step).imag))
        self._check(f(C.c_int(len(size)), _sizes(size), _strides(strides), C.c_void_p(ptr), *args), "steps")

    # indexed access (solid/src/core/cpu/template_index.c): offsets are host addresses here
    def index2(self, name, dtype, size, offsets, strides1, ptr1, strides2, ptr2):
        ptrs = (C.c_void_p * max(len(offsets), 1))(*[C.c_void_p(p) if p else None for p in offsets])
        self._check(self.fn("solid_cpu_%s_%s" % (name, dtype))(
            C.c_int(len(size)), _sizes(size), ptrs, _strides(strides1), C.c_void_p(ptr1),
            _strides(strides2), C.c_void_p(ptr2)), name)

    def fill_index(self, dtype, size, offsets, strides, ptr, value: bytes):
        ptrs = (C.c_void_p * max(len(offsets), 1))(*[C.c_void_p(p) if p else None for p in offsets])
        self._check(self.fn("solid_cpu_fill_index_%s" % dtype)(
            C.c_int(len(size)), _sizes(size), ptrs, _strides(strides), C.c_void_p(ptr), _scalar(value)), "fill_index")

    def add_if_negative(self, dtype, size, strides, ptr, value: bytes):
        self._check(self.fn("solid_cpu_add_if_negative_%s" % dtype)(
            C.c_int(len(size)), _sizes(size), _strides(strides), C.c_void_p(ptr), _scalar(value)), "add_if_negative")

    def index_to_offset(self, dtype, strides, stride_reduce, nelem, stride1, ptr1, stride2, ptr2):
        arr = (C.c_int64 * max(len(strides), 1))(*strides)
        self._check(self.fn("solid_cpu_index_to_offset_%s" % dtype)(
            C.c_int(len(strides)), arr, C.c_ssize_t(stride_reduce), C.c_size_t(nelem), C.c_ssize_t(stride1),
            C.c_void_p(ptr1), C.c_ssize_t(stride2), C.c_void_p(ptr2)), "index_to_offset")

    def gemm(self, dtype, trans_a, trans_b, m, n, k, alpha_ptr, a_ptr, lda, b_ptr, ldb, beta_ptr, c_ptr, ldc):
        """solid_cpu_gemm_<dtype> (solid/src/core/cpu/template_blas.c): integer types and bool."""
        self._check(self.fn("solid_cpu_gemm_%s" % dtype)(
            C.c_char(trans_a.encode()), C.c_char(trans_b.encode()), C.c_size_t(m), C.c_size_t(n), C.c_size_t(k),
            C.c_void_p(alpha_ptr), C.c_void_p(a_ptr), C.c_ssize_t(lda), C.c_void_p(b_ptr), C.c_ssize_t(ldb),
            C.c_void_p(beta_ptr), C.c_void_p(c_ptr), C.c_ssize_t(ldc)), "gemm")

    def byteswap(self, dtype, size, strides, ptr):
        self._check(self.fn("solid_cpu_byteswap_%s" % dtype)(
            C.c_int(len(size)), _sizes(size), _strides(strides), C.c_void_p(ptr)), "byteswap")

    def copy(self, src, dst, size1, strides1, ptr1, size2, strides2, ptr2, variant="copy"):
        self._check(self.fn("solid_cpu_%s_%s_%s" % (variant, src, dst))(
            C.c_int(len(size1)), _sizes(size1), _strides(strides1), C.c_void_p(ptr1),
            C.c_int(len(size2)), _sizes(size2), _strides(strides2), C.c_void_p(ptr2)), variant)

    def reduce_all(self, name, dtype, size, strides, ptr, bounds=(), p=None) -> bytes:
        result = (C.c_ubyte * 16)()
        args = [C.c_int(len(size)), _sizes(size), _strides(strides), C.c_void_p(ptr)]
        keep = []
        for b in bounds:
            s = _scalar(b); keep.append(s); args.append(C.byref(s))
        if p is not None:
            args.append(C.c_double(p))
        args.append(C.cast(result, C.c_void_p))
        self._check(self.fn("solid_cpu_%s_%s" % (name, dtype))(*args), name)
        return bytes(result)

    def reduce_axis(self, name, dtype, size, strides1, ptr1, strides2, ptr2, rsize, rstrides, p=None):
        args = [C.c_int(len(size)), _sizes(size)]
        if p is not None:
            args.append(C.c_double(p))
        args += [_strides(strides1), C.c_void_p(ptr1), _strides(strides2), C.c_void_p(ptr2),
                 C.c_int(len(rsize)), _sizes(rsize), _strides(rstrides)]
        self._check(self.fn("solid_cpu_%s_%s" % (name, dtype))(*args), name)


_instance = None


def get() -> SolidCPU:
    global _instance
    if _instance is None:
        _instance = SolidCPU()
    return _instance
