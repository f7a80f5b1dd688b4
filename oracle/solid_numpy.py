"""numpy restatement of the Solid CPU semantics for the elementwise / copy / reduction path.

TEST INFRASTRUCTURE: a second, independent checker beside the compiled reference
library (oracle/ref.py).  It travels to machines where the reference checkout is
absent.  Each function cites the reference code it restates.  It is pinned by
tests/test_oracle.py against (1) the compiled reference library whenever that is
available and (2) the committed golden vectors in tests/golden/, which were
produced by the reference library with tests/golden/make_golden.py.

Carriers: bool = uint8 0/1, half = uint16 bits, chalf = structured (real, imag) of
uint16 bits, cfloat/cdouble = numpy complex.  Arrays are flat (element order is the
caller's business).

Exactness: integer, bool, comparison, min/max, conversion and byte-order results
are exact; +,-,*,/ and sqrt on float/double are exact (IEEE); half results are
exact (float arithmetic followed by the reference's own rounding); library
functions (exp, sin, hypot, pow ...) agree with the reference to a few units in
the last place only, and floating-point reductions are computed in float64 here,
whereas the reference accumulates in the result type in OpenMP-thread order.
"""
from __future__ import annotations

import numpy as np

NAMES = ["bool", "uint8", "uint16", "uint32", "uint64", "int8", "int16", "int32", "int64",
         "half", "float", "double", "chalf", "cfloat", "cdouble"]
UINT = ["uint8", "uint16", "uint32", "uint64"]
SINT = ["int8", "int16", "int32", "int64"]
REAL = ["half", "float", "double"]
COMPLEX = ["chalf", "cfloat", "cdouble"]
CHALF = np.dtype([("real", "<u2"), ("imag", "<u2")])
NP = {"bool": np.uint8, "uint8": np.uint8, "uint16": np.uint16, "uint32": np.uint32, "uint64": np.uint64,
      "int8": np.int8, "int16": np.int16, "int32": np.int32, "int64": np.int64, "half": np.uint16,
      "float": np.float32, "double": np.float64, "chalf": CHALF, "cfloat": np.complex64, "cdouble": np.complex128}


# ---------------------------------------------------------------------------
# half precision: solid/src/base/generic/half.c
# ---------------------------------------------------------------------------
def half_to_float(h) -> np.ndarray:
    """half.c:26-97.  Exact, except that -0 maps to +0 (the zero test at :37-39 runs after
    the sign was stripped and returns a literal 0)."""
    h = np.asarray(h, dtype=np.uint16)
    f = h.view(np.float16).astype(np.float32)
    return np.where((h & 0x7FFF) == 0, np.float32(0), f).astype(np.float32)


def float_to_half(f) -> np.ndarray:
    """half.c:101-149.  Biased exponent < 112 -> +0; 112..143 re-biased by subtraction with the
    13 dropped bits rounded half away from zero; > 143 -> +-inf; NaN -> 0x7F00."""
    raw = np.asarray(f, dtype=np.float32).view(np.uint32)
    d = (raw & 0x007FFFFF).astype(np.int64)
    e = ((raw >> 23) & 0xFF).astype(np.int64)
    s = ((raw >> 16) & 0x8000).astype(np.int64)
    regular = (((e - 112) << 10) | (d >> 13) | s) + ((d & 0x1FFF) >= 0x1000)
    out = np.where(e < 112, 0, regular)
    out = np.where(e > 143, np.where((e == 255) & (d != 0), 0x7F00, s | 0x7C00), out)
    return (out & 0xFFFF).astype(np.uint16)


# ---------------------------------------------------------------------------
# work types (solid/include/solid/base/cpu/dtype_cpu.h:61-63) and conversion
# (solid/include/solid/base/generic/dtype_assign.h:99-163,222-288)
# ---------------------------------------------------------------------------
def _complex(re, im, npdtype) -> np.ndarray:
    """Complex array from parts without arithmetic (re + 1j*im would turn inf into nan)."""
    out = np.empty(np.shape(re), dtype=npdtype)
    out.real, out.imag = re, im
    return out


def to_work(dtype: str, x: np.ndarray) -> np.ndarray:
    if dtype == "half":
        return half_to_float(x)
    if dtype == "chalf":
        return _complex(half_to_float(x["real"]), half_to_float(x["imag"]), np.complex64)
    return np.asarray(x, dtype=NP[dtype])


def from_work(dtype: str, w: np.ndarray) -> np.ndarray:
    if dtype == "half":
        return float_to_half(np.asarray(w, dtype=np.float32))
    if dtype == "chalf":
        out = np.zeros(np.shape(w), dtype=CHALF)
        out["real"] = float_to_half(np.real(w).astype(np.float32))
        out["imag"] = float_to_half(np.imag(w).astype(np.float32))
        return out
    if dtype == "bool":
        return np.asarray(w).astype(np.uint8)
    return np.asarray(w).astype(NP[dtype])


def _real_part(dtype, x):
    if dtype == "chalf":
        return "half", x["real"]
    if dtype == "cfloat":
        return "float", np.real(x).astype(np.float32)
    if dtype == "cdouble":
        return "double", np.real(x).astype(np.float64)
    return dtype, x


def _imag_part(dtype, x):
    if dtype == "chalf":
        return "half", x["imag"]
    if dtype == "cfloat":
        return "float", np.imag(x).astype(np.float32)
    return "double", np.imag(x).astype(np.float64)


def _convert_real(src: str, dst: str, x: np.ndarray) -> np.ndarray:
    """real -> real (dtype_assign.h:109-127 with the device macros of dtype_cpu.h:68-81)."""
    if src == dst:
        return np.array(x, dtype=NP[dst])                              # raw copy
    if dst == "bool":
        if src == "half":
            return ((np.asarray(x, np.uint16) & 0x7FFF) != 0).astype(np.uint8)
        return (~(np.asarray(x) == 0)).astype(np.uint8)               # NaN -> 1
    if src == "half":
        return _convert_real("float", dst, half_to_float(x))
    if dst == "half":
        with np.errstate(over="ignore"):
            return float_to_half(np.asarray(x).astype(np.float32))     # (float)x first, then the custom rounding
    with np.errstate(invalid="ignore", over="ignore"):
        if src in ("float", "double") and dst in UINT + SINT:
            return np.trunc(np.asarray(x, dtype=np.float64)).astype(np.int64).astype(NP[dst]) \
                if dst != "uint64" else np.trunc(np.asarray(x, dtype=np.float64)).astype(np.uint64)
        return np.asarray(x).astype(NP[dst])                            # C cast


def convert(src: str, dst: str, x: np.ndarray) -> np.ndarray:
    """SOLID_ASSIGN(src, dst): complex -> real takes the real part, real -> complex sets imag = 0,
    complex -> bool is real || imag (dtype_assign.h:222-288)."""
    x = np.asarray(x, dtype=NP[src])
    if src == dst:
        return x.copy()
    if src in COMPLEX and dst in COMPLEX:
        es, re = _real_part(src, x)
        _, im = _imag_part(src, x)
        ed = {"chalf": "half", "cfloat": "float", "cdouble": "double"}[dst]
        r, i = _convert_real(es, ed, re), _convert_real(es, ed, im)
        if dst == "chalf":
            out = np.zeros(x.shape, dtype=CHALF); out["real"], out["imag"] = r, i
            return out
        return _complex(r, i, NP[dst])
    if src in COMPLEX:
        es, re = _real_part(src, x)
        if dst == "bool":
            _, im = _imag_part(src, x)
            return (_convert_real(es, "bool", re) | _convert_real(es, "bool", im)).astype(np.uint8)
        return _convert_real(es, dst, re)
    if dst in COMPLEX:
        ed = {"chalf": "half", "cfloat": "float", "cdouble": "double"}[dst]
        r = _convert_real(src, ed, x)
        if dst == "chalf":
            out = np.zeros(x.shape, dtype=CHALF); out["real"] = r
            return out
        return _complex(r, np.zeros_like(r), NP[dst])
    return _convert_real(src, dst, x)


def byteswap(dtype: str, x: np.ndarray) -> np.ndarray:
    """Reverse the bytes of each real component (dtype_assign.h:55-83,171-214)."""
    x = np.ascontiguousarray(np.asarray(x, dtype=NP[dtype]))
    comp = {"chalf": 2, "cfloat": 4, "cdouble": 8}.get(dtype, x.dtype.itemsize)
    raw = x.view(np.uint8).reshape(-1, comp)[:, ::-1]
    return np.ascontiguousarray(raw).reshape(-1).view(NP[dtype]).reshape(x.shape)


def byteswap_convert(src: str, dst: str, x: np.ndarray) -> np.ndarray:
    """SOLID_BYTESWAP_ASSIGN: swap the source element, then convert (dtype_assign.h:297-371)."""
    return convert(src, dst, byteswap(src, x))


# ---------------------------------------------------------------------------
# binary operations (solid/include/solid/core/generic/binary_ops.h:112-520)
# ---------------------------------------------------------------------------
def _promote(dtype, x):
    """C integer promotion: types narrower than int compute in int (int64 here is wide enough)."""
    return x.astype(np.int64) if dtype in ("uint8", "uint16", "int8", "int16", "int32", "uint32") else x


def _cdiv(x, y):
    """C integer division (truncation) with y != 0."""
    q = np.abs(x) // np.abs(y)
    return np.where((x < 0) != (y < 0), -q, q) if x.dtype.kind == "i" else x // y


def _cmod(x, y):
    return x - _cdiv(x, y) * y


def binary(name: str, dtype: str, x, y) -> np.ndarray:
    x = np.asarray(x, dtype=NP[dtype])
    if name in ("bitshift_left", "bitshift_right"):
        y = np.asarray(y, dtype=np.int8)
    elif name == "power" and dtype in ["bool"] + UINT + SINT:
        y = np.asarray(y, dtype=np.int16)
    else:
        y = np.asarray(y, dtype=NP[dtype])
    x, y = np.broadcast_arrays(x, y)
    if name in ("lt", "le", "ge", "gt", "eq", "ne"):
        return _compare(name, dtype, x, y)
    if dtype == "bool":
        return _binary_bool(name, x, y)
    if dtype in UINT + SINT:
        return _binary_int(name, dtype, x, y)
    if dtype in REAL:
        return _binary_real(name, dtype, x, y)
    return _binary_complex(name, dtype, x, y)


def _binary_bool(name, x, y):                                            # binary_ops.h:115-136
    table = {"add": x | y, "subtract": x & ~y & 1, "multiply": x & y, "true_divide": x & y, "divide": x & y,
             "floor_divide": x & y, "mod": np.zeros_like(x), "fmod": np.zeros_like(x),
             "bitwise_and": x & y, "bitwise_or": x | y, "bitwise_xor": x ^ y,
             "logical_and": x & y, "logical_or": x | y, "logical_xor": x ^ y,
             "min": x & y, "max": x | y, "fmin": x & y, "fmax": x | y}
    if name in table:
        return table[name].astype(np.uint8)
    if name == "power":
        return ((x != 0) | (y == 0)).astype(np.uint8)
    if name in ("bitshift_left", "bitshift_right"):
        return np.where(y == 0, x & 1, 0).astype(np.uint8)
    raise KeyError(name)


def _binary_int(name, dtype, x, y):                                      # binary_ops.h:140-262
    T = NP[dtype]
    signed = dtype in SINT
    with np.errstate(over="ignore", divide="ignore", invalid="ignore"):
        if name in ("bitshift_left", "bitshift_right"):
            xp = _promote(dtype, x); s = y.astype(np.int64)
            left = (s >= 0) if name == "bitshift_left" else (s < 0)
            n = np.abs(s)
            if dtype == "uint64":
                n = n.astype(np.uint64)
            return np.where(left, xp << n, xp >> n).astype(T)
        if name == "power":
            out = np.zeros(x.shape, dtype=T)
            for i, (b, e) in enumerate(zip(x.reshape(-1), y.reshape(-1))):
                z = T(1 if e >= 0 else 0); b = T(b); e = int(e)
                while e > 0:
                    if e & 1:
                        z = T(z * b)
                    e >>= 1
                    b = T(b * b)
                out.reshape(-1)[i] = z
            return out
        xp, yp = _promote(dtype, x), _promote(dtype, y)
        safe = np.where(yp == 0, 1, yp)
        if name == "add":
            return (xp + yp).astype(T)
        if name == "subtract":
            return (xp - yp).astype(T)
        if name == "multiply":
            return (xp * yp).astype(T)
        if name in ("bitwise_and", "bitwise_or", "bitwise_xor"):
            return {"bitwise_and": x & y, "bitwise_or": x | y, "bitwise_xor": x ^ y}[name].astype(T)
        if name in ("min", "fmin"):
            return np.where(x <= y, x, y).astype(T)
        if name in ("max", "fmax"):
            return np.where(x >= y, x, y).astype(T)
        if name == "true_divide" or (not signed and name in ("divide", "floor_divide")):
            return np.where(yp == 0, 0, _cdiv(xp, safe)).astype(T)
        if name in ("divide", "floor_divide"):                              # signed floor division, :154-203
            corr = ((xp * yp) < 0) * (yp + ((yp < 0).astype(np.int64) - (yp > 0).astype(np.int64)))
            num = xp - corr
            if name == "floor_divide":
                num = num.astype(T).astype(np.int64) if dtype != "int64" else num   # stored back into the type (:196)
            return np.where(yp == 0, 0, _cdiv(num, safe)).astype(T)
        if name == "fmod" or (not signed and name == "mod"):
            return np.where(yp == 0, 0, _cmod(xp, safe)).astype(T)
        if name == "mod":                                                   # sign of the divisor, :206-236
            z = _cmod(xp, safe)
            return np.where(yp == 0, 0, z + (((xp * yp) < 0) & (z != 0)) * yp).astype(T)
    raise KeyError(name)


def _binary_real(name, dtype, x, y):                                     # binary_ops.h:266-342
    a, b = to_work(dtype, x), to_work(dtype, y)
    W = a.dtype.type
    with np.errstate(all="ignore"):
        if name == "add":
            r = a + b
        elif name == "subtract":
            r = a - b
        elif name == "multiply":
            r = a * b
        elif name in ("divide", "true_divide"):
            r = a / b
        elif name == "floor_divide":
            r = np.floor(a / b)
        elif name == "mod":
            r = a - (np.floor(a / b) * b).astype(W)
        elif name == "fmod":
            r = np.fmod(a, b)
        elif name == "power":
            r = np.power(a.astype(np.float32), b.astype(np.float32)).astype(W)     # SOLID_DOUBLE_POW is powf
        elif name == "min":
            r = np.where(np.isnan(b) | (b < a), b, a)
        elif name == "max":
            r = np.where(np.isnan(b) | (b > a), b, a)
        elif name == "fmin":
            r = np.where(np.isnan(a) | (b <= a), b, a)
        elif name == "fmax":
            r = np.where(np.isnan(a) | (b >= a), b, a)
        else:
            raise KeyError(name)
    return from_work(dtype, r.astype(W))


def _binary_complex(name, dtype, x, y):                                  # binary_ops.h:346-520
    a, b = to_work(dtype, x), to_work(dtype, y)
    E = np.float64 if dtype == "cdouble" else np.float32
    xr, xi, yr, yi = (np.real(a).astype(E), np.imag(a).astype(E), np.real(b).astype(E), np.imag(b).astype(E))
    with np.errstate(all="ignore"):
        if name == "add":
            zr, zi = xr + yr, xi + yi
        elif name == "subtract":
            zr, zi = xr - yr, xi - yi
        elif name == "multiply":
            zr, zi = (xr * yr) - (xi * yi), (xr * yi) + (yr * xi)
        elif name in ("divide", "true_divide"):
            r = (yr * yr) + (yi * yi)
            zr, zi = ((xr * yr) + (xi * yi)) / r, ((xi * yr) - (xr * yi)) / r
        elif name in ("min", "max", "fmin", "fmax"):
            if name == "min":
                take = (np.isnan(yr) | np.isnan(yi)) | (yr < xr) | ((yr == xr) & (yi < xi))
            elif name == "max":
                take = (np.isnan(yr) | np.isnan(yi)) | (yr > xr) | ((yr == xr) & (yi > xi))
            elif name == "fmin":
                take = ((yr < xr) | np.isnan(xr)) | ((xr == yr) & ((yi < xi) | np.isnan(xi)))
            else:
                take = ((yr > xr) | np.isnan(xr)) | ((xr == yr) & ((yi > xi) | np.isnan(xi)))
            zr, zi = np.where(take, yr, xr), np.where(take, yi, xi)
        else:
            raise KeyError(name)
    return from_work(dtype, _complex(zr.astype(E), zi.astype(E), np.complex128 if dtype == "cdouble" else np.complex64))


def _compare(name, dtype, x, y):                                         # :128-133, 256-261, 310-315, 416-461
    import operator
    op = {"lt": operator.lt, "le": operator.le, "ge": operator.ge, "gt": operator.gt, "eq": operator.eq, "ne": operator.ne}[name]
    with np.errstate(invalid="ignore"):
        if dtype in COMPLEX:
            a, b = to_work(dtype, x), to_work(dtype, y)
            xr, xi, yr, yi = np.real(a), np.imag(a), np.real(b), np.imag(b)
            if name == "eq":
                return ((xr == yr) & (xi == yi)).astype(np.uint8)
            if name == "ne":
                return ((xr != yr) | (xi != yi)).astype(np.uint8)
            strict = operator.lt if name in ("lt", "le") else operator.gt
            return np.where(xr != yr, strict(xr, yr), op(xi, yi)).astype(np.uint8)
        return op(to_work(dtype, x), to_work(dtype, y)).astype(np.uint8)


# ---------------------------------------------------------------------------
# unary operations (solid/include/solid/core/generic/unary_ops.h:203-673)
# ---------------------------------------------------------------------------
_LIBM = {"sin": np.sin, "cos": np.cos, "tan": np.tan, "sinh": np.sinh, "cosh": np.cosh, "tanh": np.tanh,
         "arcsin": np.arcsin, "arccos": np.arccos, "arctan": np.arctan, "arcsinh": np.arcsinh,
         "arccosh": np.arccosh, "arctanh": np.arctanh, "sqrt": np.sqrt, "cbrt": np.cbrt, "exp": np.exp,
         "exp2": np.exp2, "expm1": np.expm1, "log": np.log, "log2": np.log2, "log10": np.log10, "log1p": np.log1p,
         "ceil": np.ceil, "floor": np.floor, "trunc": np.trunc}


def unary(name: str, dtype: str, x) -> np.ndarray:
    x = np.asarray(x, dtype=NP[dtype])
    with np.errstate(all="ignore"):
        if name in ("isinf", "isnan", "isfinite", "isposinf", "isneginf"):
            if dtype in ["bool"] + UINT + SINT:
                return np.full(x.shape, 1 if name == "isfinite" else 0, dtype=np.uint8)
            w = to_work(dtype, x)
            if dtype in COMPLEX:
                r, i = np.real(w), np.imag(w)
                return {"isinf": np.isinf(r) | np.isinf(i), "isnan": np.isnan(r) | np.isinf(i),     # sic, :660
                        "isfinite": np.isfinite(r) & np.isfinite(i)}[name].astype(np.uint8)
            return {"isinf": np.isinf(w), "isnan": np.isnan(w), "isfinite": np.isfinite(w),
                    "isposinf": (w > 0) & np.isinf(w), "isneginf": (w < 0) & np.isinf(w)}[name].astype(np.uint8)
        if dtype == "bool":
            if name in ("negative", "bitwise_not", "logical_not"):
                return (x ^ 1).astype(np.uint8)
            if name in ("fabs", "sign", "absolute"):
                return x.copy()
            raise KeyError(name)
        if dtype in UINT + SINT:
            return _unary_int(name, dtype, x)
        if dtype in REAL:
            w = to_work(dtype, x); W = w.dtype.type
            if name == "negative":
                r = -w
            elif name == "reciprocal":
                r = (1.0 / w.astype(np.float64)).astype(W)
            elif name == "square":
                r = w * w
            elif name in ("fabs", "absolute"):
                r = np.abs(w)
            elif name == "sign":
                return np.where(np.isnan(w), x, from_work(dtype, ((w > 0).astype(W) - (w < 0).astype(W))))
            elif name == "round":
                r = np.where(w >= 0, np.floor(w + W(0.5)), np.ceil(w - W(0.5)))
                r = np.where(np.abs(w) >= W(2.0) ** (23 if W is np.float32 else 52), w, r)   # already integral
                r = np.where(np.floor(w) == w, w, r)
                r = np.copysign(r, w)
            elif name == "exp10":
                r = np.exp(W(2.3025850929940459) * w)
            elif name in _LIBM:
                r = _LIBM[name](w)
            else:
                raise KeyError(name)
            return from_work(dtype, np.asarray(r).astype(W))
        return _unary_complex(name, dtype, x)


def _unary_int(name, dtype, x):
    T = NP[dtype]; signed = dtype in SINT
    if name == "negative":
        return (-1 * _promote(dtype, x)).astype(T)
    if name == "bitwise_not":
        return (~x).astype(T)
    if name == "reciprocal":
        xp = _promote(dtype, x); safe = np.where(xp == 0, 1, xp)
        return np.where(xp == 0, 0, _cdiv(np.ones_like(safe), safe)).astype(T)
    if name == "square":
        return (_promote(dtype, x) * _promote(dtype, x)).astype(T)
    if name in ("fabs", "absolute"):
        return np.where(x < 0, -_promote(dtype, x), x).astype(T) if signed else x.copy()
    if name == "sign":
        return ((x > 0).astype(np.int64) - (x < 0).astype(np.int64)).astype(T) if signed else (x > 0).astype(T)
    d = x.astype(np.float64)
    if name == "exp10":
        r = np.exp(2.3025850929940459 * d)
    else:
        r = _LIBM[name](d)
    out = np.trunc(r)
    out = np.where(np.isfinite(out), out, 0)
    res = out.astype(np.int64).astype(T) if dtype != "uint64" else out.astype(np.uint64)
    if signed and name in ("sqrt", "log", "log2", "log10"):
        res = np.where(x <= 0, 0, res).astype(T)
    if signed and name == "log1p":
        res = np.where(d <= -1, 0, res).astype(T)
    return res


def _unary_complex(name, dtype, x):
    w = to_work(dtype, x)
    E = np.float64 if dtype == "cdouble" else np.float32
    xr, xi = np.real(w).astype(E), np.imag(w).astype(E)

    def pack(zr, zi):
        out = np.empty(w.shape, dtype=w.dtype); out.real, out.imag = np.asarray(zr).astype(E), np.asarray(zi).astype(E)
        return from_work(dtype, out)

    if name == "negative":
        return pack(-xr, -xi)
    if name == "conj":
        out = pack(xr, -xi)
        if dtype == "chalf":
            out["real"] = x["real"]                                    # the real part is copied raw (:333)
        return out
    if name == "square":
        return pack((xr * xr) - (xi * xi), (E(2) * xr) * xi)
    if name == "absolute":
        return from_work({"chalf": "half", "cfloat": "float", "cdouble": "double"}[dtype], np.hypot(xr, xi).astype(E))
    if name == "fabs":
        return pack(np.hypot(xr, xi).astype(E), np.zeros_like(xr))
    if name in ("ceil", "floor", "trunc"):
        return pack(_LIBM[name](xr), _LIBM[name](xi))
    if name == "exp":
        s = np.exp(xr)
        return pack(s * np.cos(xi), s * np.sin(xi))
    if name == "log":
        s = (xr * xr) + (xi * xi)
        return pack(np.log(s) * E(0.5), np.arctan2(xi, xr))
    if name == "reciprocal":
        scale = (1.0 / ((xr * xr) + (xi * xi)).astype(np.float64)).astype(E)
        return pack(xr * scale, -(xi * scale))
    raise KeyError(name)


# ---------------------------------------------------------------------------
# reductions (solid/include/solid/core/generic/reduce_ops.h:141-1287)
# ---------------------------------------------------------------------------
def sum_type(dtype):
    return "uint64" if dtype in ["bool"] + UINT else ("int64" if dtype in SINT else dtype)


def abs_type(dtype):
    return ("u" + dtype) if dtype in SINT else {"chalf": "half", "cfloat": "float", "cdouble": "double"}.get(dtype, dtype)


def _nonzero(dtype, x):
    w = to_work(dtype, x)
    return ~(w == 0) if dtype not in COMPLEX else (~(np.real(w) == 0) | ~(np.imag(w) == 0))


def reduce_all(name: str, dtype: str, x, p: float | None = None):
    """Global reduction over a flat array; returns a numpy scalar of the result type.
    Floating-point accumulations are evaluated in float64 and rounded once."""
    x = np.asarray(x, dtype=NP[dtype]).reshape(-1)
    with np.errstate(all="ignore"):
        if name == "any":
            return np.uint8(_nonzero(dtype, x).any())
        if name == "all":
            return np.uint8(_nonzero(dtype, x).all())
        if name == "nnz":
            return np.uint64(_nonzero(dtype, x).sum())
        isint = dtype in ["bool"] + UINT + SINT
        if name in ("sum", "prod"):
            rt = sum_type(dtype)
            if isint:
                acc = x.astype(NP[rt])
                return (acc.sum(dtype=NP[rt]) if name == "sum" else acc.prod(dtype=NP[rt]))
            w = to_work(dtype, x)
            wide = w.astype(np.complex128 if dtype in COMPLEX else np.float64)
            r = wide.sum() if name == "sum" else wide.prod()
            return from_work(dtype, np.array([r]).astype(w.dtype))[0]
        if name == "sum_abs":
            if isint:
                return np.abs(x.astype(np.int64)).astype(np.uint64).sum(dtype=np.uint64) if dtype != "uint64" else x.sum(dtype=np.uint64)
            w = to_work(dtype, x)
            return from_work(abs_type(dtype), np.array([np.abs(w.astype(np.complex128 if dtype in COMPLEX else np.float64)).sum()]).astype(
                np.float64 if dtype in ("double", "cdouble") else np.float32))[0]
        if name in ("maximum", "minimum"):
            if x.size == 0:
                raise ValueError("undefined on empty tensors")
            if isint:
                return x.max() if name == "maximum" else x.min()
            if dtype in COMPLEX:
                w = to_work(dtype, x)
                order = np.lexsort((np.imag(w), np.real(w)))
                order = [i for i in order if not (np.isnan(np.real(w[i])) or np.isnan(np.imag(w[i])))]
                return x[order[-1] if name == "maximum" else order[0]] if order else x[0]
            w = to_work(dtype, x)
            if np.isnan(w).all():
                return x[0]                                                # first element is the start value
            r = np.nanmax(w) if name == "maximum" else np.nanmin(w)
            return from_work(dtype, np.array([r]).astype(w.dtype))[0]
        if name in ("maximum_abs", "minimum_abs"):
            if x.size == 0:
                raise ValueError("undefined on empty tensors")
            if isint:
                m = np.abs(x.astype(np.int64)).astype(NP[abs_type(dtype)]) if dtype in SINT and dtype != "int64" else \
                    (np.where(x < 0, (0 - x.astype(np.uint64)), x.astype(np.uint64)) if dtype == "int64" else x)
                return m.max() if name == "maximum_abs" else m.min()
            w = np.abs(to_work(dtype, x))
            r = np.nanmax(w) if name == "maximum_abs" else np.nanmin(w)
            return from_work(abs_type(dtype), np.array([r]).astype(np.float64 if dtype in ("double", "cdouble") else np.float32))[0]
        if name in ("norm2", "norm"):
            rt = "double" if isint else abs_type(dtype)
            w = to_work(dtype, x)
            sq = (np.abs(w.astype(np.complex128)) ** 2) if dtype in COMPLEX else w.astype(np.float64) ** 2
            r = np.sqrt(sq.sum()) if name == "norm2" else (sq ** (p / 2)).sum() ** (1.0 / p)
            return from_work(rt, np.array([r]).astype(np.float64 if rt == "double" else np.float32))[0]
    raise KeyError(name)


def reduce_axis(name: str, dtype: str, x: np.ndarray, axes, p=None) -> np.ndarray:
    """Reduce the given axes of an n-d array (any memory order); result in the remaining axes' order."""
    x = np.asarray(x, dtype=NP[dtype])
    axes = tuple(sorted(a % x.ndim for a in ([axes] if isinstance(axes, int) else axes)))
    keep = [i for i in range(x.ndim) if i not in axes]
    moved = np.transpose(x, keep + list(axes)).reshape([x.shape[i] for i in keep] + [-1])
    flat = moved.reshape(-1, moved.shape[-1])
    first = reduce_all(name, dtype, flat[0], p) if len(flat) else None
    out = np.zeros(len(flat), dtype=np.asarray(first).dtype if first is not None else NP[dtype])
    for i in range(len(flat)):
        out[i] = reduce_all(name, dtype, flat[i], p)
    return out.reshape([x.shape[i] for i in keep])


# ---------------------------------------------------------------------------
# fused sequences (what Ocean computes with separate kernels)
# ---------------------------------------------------------------------------
def axpy(dtype: str, a, x, y) -> np.ndarray:
    """Tensor_scale then Tensor_add (src/core/interface/tensor_itf.c:4221-4251): the product is
    rounded to the element type before the addition."""
    av = np.full(1, a).astype(NP[dtype]) if dtype != "half" else float_to_half(np.float32(a))
    prod = binary("multiply", dtype, x, np.broadcast_to(av, np.shape(x)))
    return binary("add", dtype, prod, y)


def mixed_multiply_add(ctype: str, dst: str, a, ta: str, b, tb: str, c, tc: str, swapped=(False, False, False)) -> np.ndarray:
    """dst = (dst)((ctype)a * (ctype)b + (ctype)c): each operand converted with `convert`
    (byte-reversed sources swapped first), product and sum rounded separately in ctype."""
    ops = []
    for arr, t, sw in zip((a, b, c), (ta, tb, tc), swapped):
        arr = np.asarray(arr, dtype=NP[t])
        ops.append(convert(t, ctype, byteswap(t, arr) if sw else arr))
    prod = binary("multiply", ctype, ops[0], ops[1])
    return convert(ctype, dst, binary("add", ctype, prod, ops[2]))


# ----------------------------------------------------------------------------
# ranges and indexed access
# ----------------------------------------------------------------------------
def steps(kind: str, dtype: str, n: int, offset, step) -> np.ndarray:
    """Element i = offset + i * step cast to `dtype` (solid/src/core/cpu/template_steps.c:27-92), i = 0..n-1 in
    the column-major order of the tensor.  kind 'int64': the position is a size_t, so the sum is formed in
    unsigned 64-bit arithmetic and THEN cast to the work type (negative results reach floating-point tensors as
    values near 2^64); kind 'double': product and sum in double; kind 'cdouble': both components (the real one
    only for real element types).  In-range values only for the double -> integer casts."""
    i = np.arange(n, dtype=np.uint64)
    et = {"chalf": "half", "cfloat": "float", "cdouble": "double"}.get(dtype, dtype)

    def cast_u64(u):
        if et == "bool":
            return (u & np.uint64(0xFF)).astype(np.uint8)
        if et == "half":
            return float_to_half(u.astype(np.float32))
        return u.astype(NP[et])

    def cast_double(d):
        if et == "bool":
            return (np.trunc(d).astype(np.int64) & 0xFF).astype(np.uint8)
        return _convert_real("double", et, d)

    with np.errstate(over="ignore"):
        if kind == "int64":
            u = np.uint64(int(offset) & 0xFFFFFFFFFFFFFFFF) + i * np.uint64(int(step) & 0xFFFFFFFFFFFFFFFF)
            re, im = cast_u64(u), None
        elif kind == "double":
            re, im = cast_double(np.float64(offset) + i.astype(np.float64) * np.float64(step)), None
        else:
            o, s = complex(offset), complex(step)
            re = cast_double(np.float64(o.real) + i.astype(np.float64) * np.float64(s.real))
            im = cast_double(np.float64(o.imag) + i.astype(np.float64) * np.float64(s.imag))
    if dtype not in ("chalf", "cfloat", "cdouble"):
        return re
    if im is None:
        im = np.zeros(n, dtype=NP[et])
    if dtype == "chalf":
        out = np.zeros(n, dtype=NP["chalf"]); out["real"] = re; out["imag"] = im
        return out
    return _complex(re, im, NP[dtype])


def index_offsets(size, tables, strides) -> np.ndarray:
    """Byte offset of every selected element, column-major over `size`: dimension d contributes tables[d][i]
    where it has a table and i * strides[d] otherwise (solid/include/solid/core/gpu/index2.h:288-305)."""
    off = np.zeros(1, dtype=np.int64)
    for d in range(len(size) - 1, -1, -1):
        part = np.asarray(tables[d], dtype=np.int64) if tables[d] is not None else np.arange(size[d], dtype=np.int64) * strides[d]
        off = (off[:, None] + part[None, :]).reshape(-1)
    return off


def get_index(src_bytes: np.ndarray, elemsize: int, size, tables, strides) -> np.ndarray:
    """Selected elements of a byte buffer as an (n, elemsize) byte matrix, column-major selection order."""
    off = index_offsets(size, tables, strides)
    return src_bytes[off[:, None] + np.arange(elemsize)[None, :]]


def set_index(dst_bytes: np.ndarray, elemsize: int, size, tables, strides, values: np.ndarray) -> None:
    """Scatter an (n, elemsize) byte matrix; later elements win where positions repeat."""
    off = index_offsets(size, tables, strides)
    dst_bytes[off[:, None] + np.arange(elemsize)[None, :]] = values


def add_if_negative(x: np.ndarray, value) -> np.ndarray:
    with np.errstate(over="ignore"):
        return np.where(x < 0, x + x.dtype.type(value), x).astype(x.dtype)


def index_to_offset(index: np.ndarray, strides) -> np.ndarray:
    """index[i, e] (component i of tuple e) -> sum_i strides[i] * index[i, e] as int64."""
    with np.errstate(over="ignore"):
        return (np.asarray(strides, dtype=np.int64)[:, None] * index.astype(np.int64)).sum(axis=0, dtype=np.int64)


def gemm(dtype: str, trans_a: str, trans_b: str, m: int, n: int, k: int, alpha, A, lda: int, B, ldb: int,
         beta, C, ldc: int) -> np.ndarray:
    """C = alpha * op(A) * op(B) + beta * C for the integer types and bool (solid/src/core/cpu/template_blas.c:30-314):
    column-major buffers with leading dimensions in elements, wrap-around arithmetic of the element type, and / or
    for bool.  Returns the updated copy of the C buffer."""
    npdt = NP[dtype]
    def mat(buf, rows, cols, ld):
        return np.asarray(buf).reshape(-1)[: ld * max(cols, 1)].reshape(max(cols, 1), ld).T[:rows, :cols]
    a = mat(A, m, k, lda) if trans_a in "nN" else mat(A, k, m, lda).T
    b = mat(B, k, n, ldb) if trans_b in "nN" else mat(B, n, k, ldb).T
    out = np.array(C, dtype=npdt).reshape(-1).copy()
    c = out[: ldc * max(n, 1)].reshape(max(n, 1), ldc).T[:m, :n]          # a view into `out`
    if dtype == "bool":
        prod = (a.astype(np.uint8)[:, :, None] & b.astype(np.uint8)[None, :, :]).any(axis=1).astype(np.uint8) if k else np.zeros((m, n), np.uint8)
        c[...] = (np.uint8(alpha) & prod) | (np.uint8(beta) & c)
        return out
    wide = np.uint64
    with np.errstate(over="ignore"):
        prod = a.astype(np.int64).astype(wide) @ b.astype(np.int64).astype(wide) if k else np.zeros((m, n), wide)
        res = np.int64(alpha).astype(wide) * prod + np.int64(beta).astype(wide) * c.astype(np.int64).astype(wide)
        c[...] = res.astype(npdt) if npdt in (np.uint64,) else res.astype(np.int64).astype(npdt)
    return out
