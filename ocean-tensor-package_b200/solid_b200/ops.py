"""Operations on device tensors with Ocean's names and argument meaning, dispatching
through the Solid function tables exactly as Ocean's GPU module does
(src/core/gpu/op/tensor_{unary,binary,copy,fill,reduce_all,reduce_axis}_gpu.c of the
reference): same-dtype elementwise kernels, conversion only in copy, global
reductions returning host scalars, axis reductions writing device tensors.

The mixed-dtype rules applied before dispatch mirror the interface layer
(src/core/generic/tensor_op.c:141-186): operands are brought to a common type,
broadcast with zero strides, and byte-swapped or unaligned operands are
normalised by a converting copy -- except where a fused entry point accepts them
directly.
"""
from __future__ import annotations

import builtins as _py
import struct

import numpy as np

from . import _lib
from . import _ocean
from . import dtypes as dt
from . import oplist as ol
from .tensor import Tensor


def _stream(t: Tensor) -> int:
    import torch
    return torch.cuda.current_stream(t.storage.device).cuda_stream


def _lib_for(t: Tensor):
    import torch
    torch.cuda.set_device(t.storage.device)              # Solid reads launch parameters from the current device
    return _lib.get()


def _dispatch(name: str, *args):
    """Call OcTensorGPU_<name> of the Ocean-level dispatch library; tensors become views on the
    current torch stream of their device."""
    import ctypes as C
    oc = _ocean.get()
    conv, keep = [], []
    for a in args:
        if isinstance(a, Tensor):
            v = oc.view(a, _stream(a)); keep.append(v); conv.append(C.byref(v))
        else:
            conv.append(a)
    oc._check(oc.fn(name)(*conv), name)


def scalar_bytes(value, dtype: str) -> bytes:
    """Python number -> the bytes of a solid_scalar member of `dtype` (half uses the library's own rounding)."""
    if dtype == "bool":
        return struct.pack("<B", 1 if value else 0)
    if dtype in dt.UINT or dtype in dt.SINT:
        return np.array(value).astype(dt.NUMPY[dtype]).tobytes()
    if dtype == "float":
        return struct.pack("<f", float(value))
    if dtype == "double":
        return struct.pack("<d", float(value))
    if dtype == "half":
        return _half_bits(float(value)).tobytes()
    c = complex(value)
    if dtype == "cfloat":
        return struct.pack("<ff", c.real, c.imag)
    if dtype == "cdouble":
        return struct.pack("<dd", c.real, c.imag)
    if dtype == "chalf":
        return _half_bits(c.real).tobytes() + _half_bits(c.imag).tobytes()
    raise KeyError(dtype)


def _half_bits(x: float) -> np.ndarray:
    """float -> binary16 bits, rounding half away from zero on the dropped mantissa bits
    (solid/src/base/generic/half.c:101-149)."""
    raw = np.array([x], dtype=np.float32).view(np.uint32)[0]
    d, e, s = int(raw & 0x7FFFFF), int((raw >> 23) & 0xFF), int((raw >> 16) & 0x8000)
    if e < 112:
        h = 0
    elif e > 143:
        h = 0x7F00 if (e == 255 and d) else (s | 0x7C00)
    else:
        h = (((e - 112) << 10) | (d >> 13) | s) + (1 if (d & 0x1FFF) >= 0x1000 else 0)
    return np.array([h & 0xFFFF], dtype=np.uint16)


# ---------------------------------------------------------------------------
# copy / convert
# ---------------------------------------------------------------------------
def copy(src: Tensor, dst: Tensor) -> Tensor:
    """dst[...] = src with type conversion, byte-order handling and any alignment."""
    _dispatch("copy", src, dst)
    return dst


def cast(src: Tensor, dtype: str) -> Tensor:
    return copy(src, Tensor.empty(src.size, dtype, src.storage.device))


def clone(src: Tensor) -> Tensor:
    return copy(src, Tensor.empty(src.size, src.dtype, src.storage.device))


def byteswap(t: Tensor) -> Tensor:
    """Reverse the stored bytes in place and flip the flag, so the logical values are unchanged."""
    _dispatch("byteswapNoFlag", t)
    t.byteswapped = not t.byteswapped
    return t


def fill(t: Tensor, value) -> Tensor:
    import ctypes as C
    sv = _ocean.get().scalar(scalar_bytes(value, t.dtype), t.dtype)
    _dispatch("fill", t, C.byref(sv))
    return t


def fill_nan(t: Tensor, value) -> Tensor:
    import ctypes as C
    sv = _ocean.get().scalar(scalar_bytes(value, t.dtype), t.dtype)
    _dispatch("fillNaN", t, C.byref(sv))
    return t


def masked_fill(t: Tensor, mask: Tensor, value) -> Tensor:
    import ctypes as C
    m = mask.broadcast_to(t.size)
    sv = _ocean.get().scalar(scalar_bytes(value, t.dtype), t.dtype)
    _dispatch("maskedFill", t, m, C.byref(sv))
    return t


# ---------------------------------------------------------------------------
# elementwise
# ---------------------------------------------------------------------------
_RANK = {n: i for i, n in enumerate(dt.NAMES)}


def common_type(a: str, b: str) -> str:
    """Smallest type that holds both (order of the type table; a signed/unsigned
    pair of equal width moves to the next wider signed type, integers with a
    floating type take the floating type)."""
    if a == b:
        return a
    ca, cb = a in dt.COMPLEX, b in dt.COMPLEX
    fa, fb = a in dt.GROUPS["float"], b in dt.GROUPS["float"]
    if fa or fb:
        width = max(dt.SIZE[dt.elem_type(x)] for x in (a, b) if x in dt.GROUPS["float"])
        for x in (a, b):
            if x not in dt.GROUPS["float"] and dt.SIZE[x] >= 4:
                width = max(width, 8 if dt.SIZE[x] >= 4 and width < 8 and dt.SIZE[x] > 2 else width)
        base = {2: "half", 4: "float", 8: "double"}[width]
        return {"half": "chalf", "float": "cfloat", "double": "cdouble"}[base] if (ca or cb) else base
    if a == "bool":
        return b
    if b == "bool":
        return a
    sa, sb = a in dt.SINT, b in dt.SINT
    if sa == sb:
        return a if dt.SIZE[a] >= dt.SIZE[b] else b
    s, u = (a, b) if sa else (b, a)
    if dt.SIZE[s] > dt.SIZE[u]:
        return s
    return {1: "int16", 2: "int32", 4: "int64", 8: "double"}[dt.SIZE[u]]


def _prepared(t: Tensor, dtype: str, size) -> Tensor:
    """Operand as the elementwise kernels require it: common dtype, native byte order, aligned."""
    aligned = t.ptr % t.elemsize == 0 and _py.all(s % t.elemsize == 0 for s in t.strides)
    if t.dtype != dtype or t.byteswapped or not aligned:
        t = cast(t, dtype)
    return t.broadcast_to(size)


def _broadcast_size(*tensors):
    nd = max(t.ndims for t in tensors)
    size = [1] * nd
    for t in tensors:
        own = [1] * (nd - t.ndims) + t.size
        for i, s in enumerate(own):
            if s != 1:
                if size[i] != 1 and size[i] != s:
                    raise ValueError("incompatible sizes")
                size[i] = s
    return size


def unary(name: str, src: Tensor, dst: Tensor | None = None) -> Tensor:
    if src.dtype not in dt.GROUPS[ol.UNARY_OPS[name]]:
        raise TypeError("%s is not available for type %s" % (name, src.dtype))
    x = _prepared(src, src.dtype, src.size)
    if name in ("isinf", "isnan", "isfinite", "isposinf", "isneginf"):
        rtype = "bool"
    elif name == "absolute":
        rtype = dt.elem_type(src.dtype)
    else:
        rtype = src.dtype
    out = dst if (dst is not None and dst.dtype == rtype and not dst.byteswapped) else Tensor.empty(src.size, rtype, src.storage.device)
    _dispatch(_ocean.ocean_name(name), x, out)
    if dst is not None and out is not dst:
        copy(out, dst)
        return dst
    return out


def binary(name: str, a: Tensor, b: Tensor, dst: Tensor | None = None) -> Tensor:
    size = _broadcast_size(a, b)
    # shifts keep the type of the shifted tensor (the count is cast to int8); every other
    # operation works in the common type of both operands
    ctype = a.dtype if name in ("bitshift_left", "bitshift_right") else common_type(a.dtype, b.dtype)
    if name == "power" and a.dtype in dt.GROUPS["integer_bool"] and b.dtype in dt.GROUPS["integer_bool"]:
        ctype = a.dtype                                  # integer base with an integer exponent (cast to int16)
    if ctype not in dt.GROUPS[ol.BINARY_OPS[name]]:
        raise TypeError("%s is not available for type %s" % (name, ctype))
    x = _prepared(a, ctype, size)
    if name in ("bitshift_left", "bitshift_right"):
        y = _prepared(b, "int8", size)
    elif name == "power" and ctype in dt.GROUPS["integer_bool"]:
        y = _prepared(b, "int16", size)
    else:
        y = _prepared(b, ctype, size)
    rtype = "bool" if name in ol.COMPARE_OPS else ctype
    out = dst if (dst is not None and dst.dtype == rtype and not dst.byteswapped and dst.size == size) \
        else Tensor.empty(size, rtype, a.storage.device)
    _dispatch(_ocean.ocean_name(name), x, y, out)
    if dst is not None and out is not dst:
        copy(out, dst)
        return dst
    return out


def scalar_op(name: str, a: Tensor, value, dst: Tensor | None = None) -> Tensor:
    """Tensor (op) Python scalar in the tensor's own type with the scalar passed by value (Ocean's
    addScalar, subtractScalar, multiplyScalar, bitwise{And,Or,Xor}Scalar without the 0-d device tensor)."""
    if name not in ol.SCALAR_OPS or a.dtype not in dt.GROUPS[ol.SCALAR_OPS[name]]:
        raise TypeError("%s with a scalar is not available for type %s" % (name, a.dtype))
    x = _native(a)
    out = dst if (dst is not None and dst.dtype == a.dtype and not dst.byteswapped and dst.size == a.size) \
        else Tensor.empty(a.size, a.dtype, a.storage.device)
    sv = _ocean.get().scalar(scalar_bytes(value, a.dtype), a.dtype)
    import ctypes as C
    _dispatch(_ocean.ocean_name(name) + "Scalar" if name != "multiply" else "multiplyScalar", x, C.byref(sv), out)
    if dst is not None and out is not dst:
        copy(out, dst)
        return dst
    return out


def add(a, b, dst=None):
    return binary("add", a, b, dst)


def subtract(a, b, dst=None):
    return binary("subtract", a, b, dst)


def scale(a, b, dst=None):
    """Elementwise product (Ocean's `scale`; `*` is matrix multiplication there)."""
    return binary("multiply", a, b, dst)


def divide(a, b, dst=None):
    return binary("divide", a, b, dst)


for _n in ol.UNARY_OPS:
    if _n not in globals():
        globals()[_n] = (lambda n: (lambda src, dst=None: unary(n, src, dst)))(_n)
del _n


def axpy(a, x: Tensor, y: Tensor, dst: Tensor | None = None) -> Tensor:
    """a*x + y in the element type with the product rounded first (fused multiplyScalar + add)."""
    size = _broadcast_size(x, y)
    xx, yy = _prepared(x, x.dtype, size), _prepared(y, x.dtype, size)
    out = dst or Tensor.empty(size, x.dtype, x.storage.device)
    _lib_for(out).axpy(x.dtype, size, scalar_bytes(a, x.dtype), xx.strides, xx.ptr, yy.strides, yy.ptr,
                       out.strides, out.ptr, _stream(out))
    return out


def multiply_add(a: Tensor, b: Tensor, c: Tensor, dst: Tensor, ctype: str | None = None) -> Tensor:
    """dst = a*b + c in one kernel, operands in their own dtype / byte order / alignment.
    `ctype` defaults to the type Ocean would promote (a, b, c) to."""
    ctype = ctype or common_type(common_type(a.dtype, b.dtype), c.dtype)
    if ctype in dt.COMPLEX:
        raise TypeError("multiply_add computes in float or double")
    ctype = "double" if ctype not in ("float", "half") else "float"
    size = dst.size
    ops_ = [(t.broadcast_to(size)) for t in (a, b, c)] + [dst]
    _lib_for(dst).mixed_multiply_add(size, [(t.ptr, t.strides, t.dtype, t.byteswapped) for t in ops_], ctype, _stream(dst))
    return dst


# ---------------------------------------------------------------------------
# reductions
# ---------------------------------------------------------------------------
_scratch = {}


def _scratch_buffer(device, nbytes: int):
    import torch
    key = (device, )
    buf = _scratch.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _scratch[key] = buf
    return buf


def _native(t: Tensor) -> Tensor:
    aligned = t.ptr % t.elemsize == 0 and _py.all(s % t.elemsize == 0 for s in t.strides)
    return clone(t) if (t.byteswapped or not aligned) else t


def reduce_all(name: str, t: Tensor, bounds=(), p=None):
    """Global reduction; returns a numpy scalar of the result type (on the host, like Ocean)."""
    import ctypes as C
    t = _native(t)
    oc = _ocean.get()
    oname = _ocean.ocean_name(name)
    if name in ol.REDUCE_BOOL_OPS:
        r = C.c_int(0)
        _dispatch(oname, t, C.byref(r))
        return np.uint8(r.value)
    if name in ol.REDUCE_BOUND1_OPS or name in ol.REDUCE_BOUND2_OPS:
        r = C.c_int(0)
        sv = [oc.scalar(scalar_bytes(b, t.dtype), t.dtype) for b in bounds]
        _dispatch(oname, t, *[C.byref(v) for v in sv], C.byref(r))
        return np.uint8(r.value)
    if name in ol.REDUCE_U64_OPS:
        r = C.c_uint64(0)
        _dispatch(oname, t, C.byref(r))
        return np.uint64(r.value)
    res = _ocean.ScalarView()
    if name in ol.REDUCE_NORM_OPS:
        _dispatch(oname, t, C.c_double(p), C.byref(res))
    else:
        _dispatch(oname, t, C.byref(res))
    rtype = dt.NAMES[res.dtype]
    raw = bytes(C.string_at(C.addressof(res.value), 16))
    return np.frombuffer(raw[: dt.SIZE[rtype]], dtype=dt.NUMPY[rtype])[0]


def reduce_axis(name: str, t: Tensor, axes, dst: Tensor | None = None, p=None, keepdims: bool = False) -> Tensor:
    import ctypes as C
    t = _native(t)
    axes = sorted({a % t.ndims for a in ([axes] if isinstance(axes, int) else axes)})
    keep = [i for i in range(t.ndims) if i not in axes]
    rtype = ol.reduce_result_type("axis_" + name, t.dtype)
    osize = [t.size[i] for i in keep]
    out = dst if dst is not None else Tensor.empty(osize, rtype, t.storage.device)
    ax = (C.c_int * max(len(axes), 1))(*axes)
    oname = _ocean.ocean_name("axis_" + name)
    if p is None:
        _dispatch(oname, t, C.c_int(len(axes)), ax, out)
    else:
        _dispatch(oname, t, C.c_double(p), C.c_int(len(axes)), ax, out)
    if keepdims:
        size = [1 if i in axes else t.size[i] for i in range(t.ndims)]
        return Tensor(out.storage, out.dtype, size, None, out.offset)
    return out


def _reduction(name):
    def run(t: Tensor, axes=None, dst=None, keepdims=False):
        if axes is None:
            return reduce_all(name, t)
        return reduce_axis(name, t, axes, dst, keepdims=keepdims)
    run.__name__ = name
    return run


sum = _reduction("sum")
prod = _reduction("prod")
any = _reduction("any")
all = _reduction("all")
nnz = _reduction("nnz")
maximum = _reduction("maximum")
minimum = _reduction("minimum")
sum_abs = _reduction("sum_abs")
maximum_abs = _reduction("maximum_abs")
minimum_abs = _reduction("minimum_abs")
norm2 = _reduction("norm2")


def norm(t: Tensor, p=2, axes=None, dst=None):
    """p-norm with Ocean's special cases (src/core/interface/tensor_itf.c:5405-5447):
    p=0 counts non-zeros, 1 sums magnitudes, inf takes the largest magnitude, 2 is norm2."""
    name, kw = {0: ("nnz", {}), 1: ("sum_abs", {}), 2: ("norm2", {}), float("inf"): ("maximum_abs", {})}.get(p, ("norm", {"p": float(p)}))
    if axes is None:
        return reduce_all(name, t, **kw)
    return reduce_axis(name, t, axes, dst, **kw)


def axpy_sums(a, x: Tensor, y: Tensor, z: Tensor | None = None, sums=None):
    """Fused z = a*x + y with sum(z) and sum(z*z) left on the device: returns (z, sums) where
    sums is a 2-element torch tensor {sum(z), sum(z*z)} of the element type.  Contiguous float/double."""
    import torch
    if not (x.is_contiguous() and y.is_contiguous()) or x.dtype not in ("float", "double") or x.dtype != y.dtype:
        raise TypeError("axpy_sums takes contiguous float or double tensors of one type")
    lib = _lib_for(x)
    z = z or Tensor.empty(x.size, x.dtype, x.storage.device)
    tdt = torch.float32 if x.dtype == "float" else torch.float64
    if sums is None:
        sums = torch.empty(2, dtype=tdt, device=x.storage.device)
    part = _scratch_buffer(x.storage.device, lib.axpy_sums_buffer_size(x.device_index, x.nelem))
    lib.axpy_sums(x.dtype, x.nelem, scalar_bytes(a, x.dtype), x.ptr, y.ptr, z.ptr, sums.data_ptr(), part.data_ptr(), _stream(x))
    return z, sums


# ----------------------------------------------------------------------------
# indexed access (Ocean's tensor[index] with integer index lists)
# ----------------------------------------------------------------------------
def _index_view(t: Tensor, positions):
    """OcIndexView for `t` and one entry per dimension: None (every position, by stride) or a sequence of integer
    positions (negative ones count from the end).  Returns the view, the selection shape and the objects to keep."""
    import ctypes as C
    oc = _ocean.get()
    if len(positions) != t.ndims:
        raise ValueError("one index entry per dimension is needed")
    ix = _ocean.IndexView()
    ix.view = oc.view(t, _stream(t))
    ix.ndims = t.ndims
    keep, shape = [], []
    for d, pos in enumerate(positions):
        if pos is None:
            ix.size[d] = t.size[d]; shape.append(t.size[d])
            continue
        p = np.asarray(pos, dtype=np.int64).reshape(-1)
        p = np.where(p < 0, p + t.size[d], p)
        if p.size and (p.min() < 0 or p.max() >= t.size[d]):
            raise IndexError("index out of range in dimension %d" % d)
        table = Tensor.from_numpy(p * t.strides[d], "int64", t.storage.device)
        tv = oc.view(table, _stream(t))
        keep += [table, tv]
        ix.offsets[d] = C.pointer(tv)
        ix.size[d] = p.size; shape.append(int(p.size))
    return ix, shape, keep


def take(t: Tensor, positions, dst: Tensor | None = None) -> Tensor:
    """dst = t[positions] (outer product of the per-dimension index lists)."""
    import ctypes as C
    t = _native(t)
    ix, shape, keep = _index_view(t, positions)
    out = dst if dst is not None else Tensor.empty(shape, t.dtype, t.storage.device)
    _dispatch("getIndex", C.byref(ix), out)
    return out


def put(t: Tensor, positions, src: Tensor) -> Tensor:
    """t[positions] = src (positions must not repeat)."""
    import ctypes as C
    ix, shape, keep = _index_view(t, positions)
    _dispatch("setIndex", C.byref(ix), _native(src) if src.dtype == t.dtype else cast(src, t.dtype))
    return t


def fill_at(t: Tensor, positions, value) -> Tensor:
    """t[positions] = value."""
    import ctypes as C
    ix, shape, keep = _index_view(t, positions)
    sv = _ocean.get().scalar(scalar_bytes(value, t.dtype), t.dtype)
    _dispatch("fillIndex", C.byref(ix), C.byref(sv))
    return t
