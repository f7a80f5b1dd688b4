"""ctypes binding of libsolid_core_gpu.so (the C-ABI declared in include/solid_core_gpu.h).

There is no fallback: if the library has not been built, importing this module
raises.  Pointers are plain integers (device addresses), sizes and strides are
Python sequences; strides are in bytes.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

from . import dtypes as dt
from . import oplist as ol

LIB_PATH = Path(__file__).resolve().parent.parent / "lib" / "libsolid_core_gpu.so"


class SolidError(RuntimeError):
    """A Solid entry point returned -1; the message is the library's solid_errmsg."""


class Scalar(C.Structure):
    """solid_scalar passed BY VALUE (solid/include/solid/base/generic/scalar.h:27-43): a 16-byte union.
    The x86-64 calling convention classifies its first eight bytes as INTEGER (the integer members
    overlap the floating ones there) and its second eight bytes as SSE (only cdouble.imag lives
    there), so it travels in one general and one vector register.  ctypes cannot pass unions by
    value; a struct {uint64, double} has exactly that classification."""
    _fields_ = [("lo", C.c_uint64), ("hi", C.c_double)]


class Dim3(C.Structure):
    _fields_ = [("x", C.c_uint), ("y", C.c_uint), ("z", C.c_uint)]


class ReduceAxisData(C.Structure):
    _fields_ = [("size", C.c_size_t * 8), ("rsize", C.c_size_t * 8),
                ("strides1", C.c_ssize_t * 8), ("strides2", C.c_ssize_t * 8), ("rstrides", C.c_ssize_t * 8),
                ("ptr1", C.c_void_p), ("ptr2", C.c_void_p), ("ptrBuffer", C.c_void_p),
                ("nelem", C.c_size_t), ("relem", C.c_size_t), ("ndims", C.c_int), ("rdims", C.c_int)]


class ReduceAxisConfig(C.Structure):
    _fields_ = [("data", ReduceAxisData), ("mode", C.c_int),
                ("gridSize", Dim3), ("blockSize", Dim3), ("gridSizeFinalize", Dim3), ("blockSizeFinalize", Dim3),
                ("bufferSize", C.c_size_t), ("sharedMem", C.c_size_t), ("sharedMemFinalize", C.c_size_t),
                ("stream", C.c_void_p)]


class Operand(C.Structure):
    """solid_gpu_operand of the mixed-dtype fused entry points."""
    _fields_ = [("ptr", C.c_void_p), ("strides", C.POINTER(C.c_ssize_t)), ("dtype", C.c_int),
                ("byteswapped", C.c_int)]


def _sizes(seq):
    return (C.c_size_t * max(len(seq), 1))(*seq)


def _strides(seq):
    return (C.c_ssize_t * max(len(seq), 1))(*seq)


def _pointers(seq):
    return (C.c_void_p * max(len(seq), 1))(*[C.c_void_p(p) if p else None for p in seq])


class CDouble(C.Structure):
    """solid_cdouble, passed by value to the steps_cdouble functions."""
    _fields_ = [("real", C.c_double), ("imag", C.c_double)]


def scalar_from_bytes(raw: bytes) -> Scalar:
    s = Scalar()
    C.memmove(C.addressof(s), raw, min(len(raw), 16))
    return s


class SolidGPU:
    """Thin, typed access to every exported entry point."""

    def __init__(self, path: Path | str = LIB_PATH):
        path = Path(path)
        if not path.exists():
            raise ImportError("%s is missing: build it with ocean-tensor-package_b200/build.py "
                              "(there is no CPU fallback)" % path)
        self.path = path
        self.dll = C.CDLL(str(path), mode=C.RTLD_GLOBAL)
        self.dll.solid_gpu_initialize.restype = C.c_int

    # -- helpers ---------------------------------------------------------------
    def errmsg(self) -> str:
        p = C.c_char_p.in_dll(self.dll, "solid_errmsg")
        return (p.value or b"").decode(errors="replace")

    def _check(self, status: int, what: str):
        if status != 0:
            raise SolidError("%s: %s" % (what, self.errmsg()))

    def fn(self, name: str):
        f = getattr(self.dll, name)
        f.restype = C.c_int
        return f

    def has(self, name: str) -> bool:
        return hasattr(self.dll, name)

    def initialize(self):
        self._check(self.dll.solid_gpu_initialize(), "solid_gpu_initialize")

    # -- elementwise -------------------------------------------------------------
    def fill(self, name, dtype, size, strides, ptr, value: bytes, stream=0):
        f = self.fn("solid_gpu_%s_%s" % (name, dtype))
        self._check(f(C.c_int(len(size)), _sizes(size), _strides(strides), C.c_void_p(ptr),
                      scalar_from_bytes(value), C.c_void_p(stream)), "%s_%s" % (name, dtype))

    def masked_fill(self, dtype, size, strides1, ptr1, strides2, ptr2, value: bytes, stream=0):
        f = self.fn("solid_gpu_masked_fill_%s" % dtype)
        self._check(f(C.c_int(len(size)), _sizes(size), _strides(strides1), C.c_void_p(ptr1),
                      _strides(strides2), C.c_void_p(ptr2), scalar_from_bytes(value), C.c_void_p(stream)),
                    "masked_fill_%s" % dtype)

    def unary(self, name, dtype, size, strides1, ptr1, strides2, ptr2, stream=0):
        f = self.fn("solid_gpu_%s_%s" % (name, dtype))
        self._check(f(C.c_int(len(size)), _sizes(size), _strides(strides1), C.c_void_p(ptr1),
                      _strides(strides2), C.c_void_p(ptr2), C.c_void_p(stream)), "%s_%s" % (name, dtype))

    def binary(self, name, dtype, size, strides1, ptr1, strides2, ptr2, strides3, ptr3, stream=0):
        f = self.fn("solid_gpu_%s_%s" % (name, dtype))
        self._check(f(C.c_int(len(size)), _sizes(size), _strides(strides1), C.c_void_p(ptr1),
                      _strides(strides2), C.c_void_p(ptr2), _strides(strides3), C.c_void_p(ptr3),
                      C.c_void_p(stream)), "%s_%s" % (name, dtype))

    def scalar_op(self, name, dtype, size, strides1, ptr1, value: bytes, strides2, ptr2, stream=0):
        """dst = op(src, value) with the scalar passed by value; name is 'add', 'subtract', 'multiply',
        'bitwise_and', 'bitwise_or' or 'bitwise_xor'."""
        f = self.fn("solid_gpu_%s_scalar_%s" % (name, dtype))
        st2 = _strides(strides2) if strides2 is not None else None          # None, None: in place
        self._check(f(C.c_int(len(size)), _sizes(size), _strides(strides1), C.c_void_p(ptr1), scalar_from_bytes(value),
                      st2, C.c_void_p(ptr2), C.c_void_p(stream)), "%s_scalar_%s" % (name, dtype))

    def steps(self, kind, dtype, size, strides, ptr, offset, step, stream=0):
        """tensor[i] = offset + i * step; kind is 'int64', 'double' or 'cdouble' (complex element types only)."""
        f = self.fn("solid_gpu_steps_%s_%s" % (kind, dtype))
        if kind == "int64":
            args = (C.c_int64(int(offset)), C.c_int64(int(step)))
        elif kind == "double":
            args = (C.c_double(float(offset)), C.c_double(float(step)))
        else:
            args = (CDouble(complex(offset).real, complex(offset).imag), CDouble(complex(step).real, complex(step).imag))
        self._check(f(C.c_int(len(size)), _sizes(size), _strides(strides), C.c_void_p(ptr), *args, C.c_void_p(stream)),
                    "steps_%s_%s" % (kind, dtype))

    def unary_checked(self, name, dtype, size, strides1, ptr1, strides2, ptr2, flag_ptr, stream=0):
        """solid_gpu_<name>_checked_<dtype>: the unary function plus a device int flag set when an element lies
        outside the function's real domain."""
        f = self.fn("solid_gpu_%s_checked_%s" % (name, dtype))
        st2 = _strides(strides2) if strides2 is not None else None
        self._check(f(C.c_int(len(size)), _sizes(size), _strides(strides1), C.c_void_p(ptr1), st2, C.c_void_p(ptr2),
                      C.c_void_p(flag_ptr), C.c_void_p(stream)), "%s_checked_%s" % (name, dtype))

    def gemm(self, dtype, trans_a, trans_b, m, n, k, alpha_ptr, a_ptr, lda, b_ptr, ldb, beta_ptr, c_ptr, ldc,
             scalars_on_host=True, stream=0):
        """C = alpha * op(A) * op(B) + beta * C for the integer types and bool; leading dimensions in elements;
        alpha_ptr / beta_ptr are host addresses (scalars_on_host) or device addresses, None for 1 and 0."""
        f = self.fn("solid_gpu_gemm_%s" % dtype)
        self._check(f(C.c_char(trans_a.encode()), C.c_char(trans_b.encode()), C.c_size_t(m), C.c_size_t(n), C.c_size_t(k),
                      C.c_void_p(alpha_ptr), C.c_void_p(a_ptr), C.c_ssize_t(lda), C.c_void_p(b_ptr), C.c_ssize_t(ldb),
                      C.c_void_p(beta_ptr), C.c_void_p(c_ptr), C.c_ssize_t(ldc), C.c_int(1 if scalars_on_host else 0),
                      C.c_void_p(stream)), "gemm_%s" % dtype)

    # -- indexed access ----------------------------------------------------------------
    def index2(self, name, dtype, size, offsets, strides1, ptr1, strides2, ptr2, stream=0):
        """name 'get_index' (ptr2 = ptr1[index]) or 'set_index' (ptr1[index] = ptr2); offsets: per dimension a
        device address of int64 byte offsets, or None where the dimension is addressed by strides1."""
        f = self.fn("solid_gpu_%s_%s" % (name, dtype))
        self._check(f(C.c_int(len(size)), _sizes(size), _pointers(offsets), _strides(strides1), C.c_void_p(ptr1),
                      _strides(strides2), C.c_void_p(ptr2), C.c_void_p(stream)), "%s_%s" % (name, dtype))

    def fill_index(self, dtype, size, offsets, strides, ptr, value: bytes, stream=0):
        f = self.fn("solid_gpu_fill_index_%s" % dtype)
        self._check(f(C.c_int(len(size)), _sizes(size), _pointers(offsets), _strides(strides), C.c_void_p(ptr),
                      scalar_from_bytes(value), C.c_void_p(stream)), "fill_index_%s" % dtype)

    def add_if_negative(self, dtype, size, strides, ptr, value: bytes, stream=0):
        f = self.fn("solid_gpu_add_if_negative_%s" % dtype)
        self._check(f(C.c_int(len(size)), _sizes(size), _strides(strides), C.c_void_p(ptr), scalar_from_bytes(value),
                      C.c_void_p(stream)), "add_if_negative_%s" % dtype)

    def index_to_offset(self, dtype, strides, stride_reduce, nelem, stride1, ptr1, stride2, ptr2, stream=0):
        f = self.fn("solid_gpu_index_to_offset_%s" % dtype)
        arr = (C.c_int64 * max(len(strides), 1))(*strides)
        self._check(f(C.c_int(len(strides)), arr, C.c_ssize_t(stride_reduce), C.c_size_t(nelem), C.c_ssize_t(stride1),
                      C.c_void_p(ptr1), C.c_ssize_t(stride2), C.c_void_p(ptr2), C.c_void_p(stream)),
                    "index_to_offset_%s" % dtype)

    def axpy(self, dtype, size, a: bytes, strides1, ptr1, strides2, ptr2, strides3, ptr3, stream=0):
        f = self.fn("solid_gpu_axpy_%s" % dtype)
        self._check(f(C.c_int(len(size)), _sizes(size), scalar_from_bytes(a), _strides(strides1), C.c_void_p(ptr1),
                      _strides(strides2), C.c_void_p(ptr2), _strides(strides3), C.c_void_p(ptr3),
                      C.c_void_p(stream)), "axpy_%s" % dtype)

    def byteswap(self, dtype, size, strides, ptr, stream=0):
        f = self.fn("solid_gpu_byteswap_%s" % dtype)
        self._check(f(C.c_int(len(size)), _sizes(size), _strides(strides), C.c_void_p(ptr), C.c_void_p(stream)),
                    "byteswap_%s" % dtype)

    def copy(self, src, dst, size1, strides1, ptr1, size2, strides2, ptr2, stream=0, variant="copy"):
        """variant: 'copy', 'byteswap_copy' (source bytes reversed) or 'copy_regular' (one shape)."""
        f = self.fn("solid_gpu_%s_%s_%s" % (variant, src, dst))
        if variant == "copy_regular":
            st = f(C.c_int(len(size1)), _sizes(size1), _strides(strides1), C.c_void_p(ptr1),
                   _strides(strides2), C.c_void_p(ptr2), C.c_void_p(stream))
        else:
            st = f(C.c_int(len(size1)), _sizes(size1), _strides(strides1), C.c_void_p(ptr1),
                   C.c_int(len(size2)), _sizes(size2), _strides(strides2), C.c_void_p(ptr2), C.c_void_p(stream))
        self._check(st, "%s_%s_%s" % (variant, src, dst))

    def copy_ex(self, src, dst, flags, size1, strides1, ptr1, size2, strides2, ptr2, stream=0):
        f = self.fn("solid_gpu_copy_ex")
        self._check(f(C.c_int(dt.INDEX[src]), C.c_int(dt.INDEX[dst]), C.c_int(flags),
                      C.c_int(len(size1)), _sizes(size1), _strides(strides1), C.c_void_p(ptr1),
                      C.c_int(len(size2)), _sizes(size2), _strides(strides2), C.c_void_p(ptr2),
                      C.c_void_p(stream)), "copy_ex %s->%s" % (src, dst))

    # -- reductions ----------------------------------------------------------------
    def reduce_all_buffer_size(self, nelem: int, device: int) -> int:
        out = C.c_size_t(0)
        self._check(self.fn("solid_gpu_reduce_all_buffer_size")(C.c_size_t(nelem), C.c_int(device), C.byref(out)),
                    "reduce_all_buffer_size")
        return out.value

    def reduce_all(self, name, dtype, size, strides, ptr, buffer, stream=0, bounds=(), p=None) -> bytes:
        """Run a global reduction; returns the 16 raw result bytes (host)."""
        f = self.fn("solid_gpu_%s_%s" % (name, dtype))
        result = (C.c_ubyte * 16)()
        args = [C.c_int(len(size)), _sizes(size), _strides(strides), C.c_void_p(ptr)]
        keep = []
        for b in bounds:
            s = scalar_from_bytes(b); keep.append(s); args.append(C.byref(s))
        if p is not None:
            args.append(C.c_double(p))
        args += [C.cast(result, C.c_void_p), C.c_void_p(buffer), C.c_void_p(stream)]
        self._check(f(*args), "%s_%s" % (name, dtype))
        return bytes(result)

    def reduce_all_device(self, name, dtype, size, strides, ptr, result_ptr, buffer, stream=0):
        f = self.fn("solid_gpu_reduce_all_device")
        self._check(f(C.c_char_p(name.encode()), C.c_int(dt.INDEX[dtype]), C.c_int(len(size)), _sizes(size),
                      _strides(strides), C.c_void_p(ptr), C.c_void_p(result_ptr), C.c_void_p(buffer),
                      C.c_void_p(stream)), "reduce_all_device %s %s" % (name, dtype))

    def reduce_axis_prepare(self, elemsize, size, strides1, ptr1, strides2, ptr2, rsize, rstrides, stream=0):
        cfg = ReduceAxisConfig()
        f = self.fn("solid_gpu_reduce_axis_prepare")
        self._check(f(C.byref(cfg), C.c_int(elemsize), C.c_int(len(size)), _sizes(size), _strides(strides1),
                      C.c_void_p(ptr1), _strides(strides2), C.c_void_p(ptr2), C.c_int(len(rsize)), _sizes(rsize),
                      _strides(rstrides), C.c_void_p(stream)), "reduce_axis_prepare")
        return cfg

    def reduce_axis(self, name, dtype, cfg: ReduceAxisConfig, p=None):
        f = self.fn("solid_gpu_%s_%s" % (name, dtype))
        st = f(C.byref(cfg)) if p is None else f(C.byref(cfg), C.c_double(p))
        self._check(st, "%s_%s" % (name, dtype))

    def noalloc_scratch_size(self) -> int:
        f = self.dll.solid_gpu_noalloc_scratch_size
        f.restype = C.c_int
        return f()

    def axis_sum_float_noalloc(self, cfg: ReduceAxisConfig):
        """Float axis sum that uses the scratch array built into the library (allocates nothing)."""
        self._check(self.fn("solid_gpu_axis_sum_float_noalloc")(C.byref(cfg)), "axis_sum_float_noalloc")

    # -- fused -----------------------------------------------------------------------
    def axpy_sums_buffer_size(self, device: int, n: int) -> int:
        out = C.c_size_t(0)
        self._check(self.fn("solid_gpu_axpy_sums_buffer_size")(C.c_int(device), C.c_size_t(n), C.byref(out)), "axpy_sums_buffer_size")
        return out.value

    def axpy_sums(self, dtype, n, a: bytes, x, y, z, sums, partials, stream=0):
        f = self.fn("solid_gpu_axpy_sums_%s" % dtype)
        self._check(f(C.c_size_t(n), scalar_from_bytes(a), C.c_void_p(x), C.c_void_p(y), C.c_void_p(z),
                      C.c_void_p(sums), C.c_void_p(partials), C.c_void_p(stream)), "axpy_sums_%s" % dtype)

    def peer_sum_buffer_size(self, world: int) -> int:
        out = C.c_size_t(0)
        self._check(self.fn("solid_gpu_peer_sum_buffer_size")(C.c_int(world), C.byref(out)), "peer_sum_buffer_size")
        return out.value

    def peer_sum_float(self, world, rank, buffers, sequence, count, local, result, sqrt_mask=0, limit_us=0,
                       status=0, stream=0):
        """buffers: device addresses of every rank's exchange buffer as mapped in this process."""
        arr = (C.c_void_p * world)(*[C.c_void_p(int(b)) for b in buffers])
        self._check(self.fn("solid_gpu_peer_sum_float")(C.c_int(world), C.c_int(rank), arr, C.c_uint(sequence), C.c_int(count),
                                                        C.c_void_p(local), C.c_void_p(result), C.c_int(sqrt_mask),
                                                        C.c_uint(limit_us), C.c_void_p(status), C.c_void_p(stream)),
                    "peer_sum_float")

    def mixed_multiply_add(self, size, operands, ctype, stream=0):
        """operands: four tuples (ptr, strides, dtype name, byteswapped) for a, b, c, dst."""
        ops, keep = [], []
        for ptr, strides, dtype, swapped in operands:
            st = _strides(strides); keep.append(st)
            ops.append(Operand(C.c_void_p(ptr), C.cast(st, C.POINTER(C.c_ssize_t)), dt.INDEX[dtype], int(bool(swapped))))
        f = self.fn("solid_gpu_mixed_multiply_add")
        self._check(f(C.c_int(len(size)), _sizes(size), C.byref(ops[0]), C.byref(ops[1]), C.byref(ops[2]),
                      C.byref(ops[3]), C.c_int(dt.INDEX[ctype]), C.c_void_p(stream)), "mixed_multiply_add")


_instance: SolidGPU | None = None


def get() -> SolidGPU:
    global _instance
    if _instance is None:
        _instance = SolidGPU()
    return _instance
