"""Shared helpers of the parity tests: seeded data per element type, tensor views
described as (byte offset, sizes, byte strides) over a flat buffer, device
mirrors of host buffers, and comparison with the tolerance each class of
operation is held to."""
from __future__ import annotations

import numpy as np

from solid_b200 import dtypes as dt


# ----------------------------------------------------------------------------
# data
# ----------------------------------------------------------------------------
def f32_to_solid_half(x: np.ndarray) -> np.ndarray:
    """float32 -> binary16 bits with the rounding of solid/src/base/generic/half.c:101-149
    (round half away from zero on the dropped bits, no subnormals)."""
    raw = np.asarray(x, dtype=np.float32).view(np.uint32)
    d = raw & 0x007FFFFF
    e = (raw >> 23) & 0xFF
    s = ((raw >> 16) & 0x8000).astype(np.uint32)
    h = (((e.astype(np.int64) - 112) << 10) | (d >> 13) | s).astype(np.int64)
    h = h + ((d & 0x1FFF) >= 0x1000)
    out = np.where(e < 112, 0, h)
    big = e > 143
    out = np.where(big, np.where((e == 255) & (d != 0), 0x7F00, s | 0x7C00), out)
    return out.astype(np.uint16)


def random_values(dtype: str, n: int, rng: np.random.Generator, kind: str = "general") -> np.ndarray:
    """n seeded elements of `dtype` as its numpy carrier.
    kind: 'general' (signed, moderate), 'positive' (0.01..10), 'unit' (-1..1), 'small' (tiny ints),
          'special' (general plus inf/nan/zeros for floating types)."""
    npdt = dt.NUMPY[dtype]
    if dtype == "bool":
        return (rng.random(n) < 0.5).astype(np.uint8)
    if dtype in dt.UINT:
        hi = {"general": 120, "positive": 120, "unit": 2, "small": 12, "special": 120}[kind]
        return rng.integers(1 if kind == "positive" else 0, hi, n).astype(npdt)
    if dtype in dt.SINT:
        hi = {"general": 100, "positive": 100, "unit": 2, "small": 12, "special": 100}[kind]
        lo = 1 if kind == "positive" else -hi
        return rng.integers(lo, hi, n).astype(npdt)

    def reals(m):
        if kind == "positive":
            v = rng.uniform(0.01, 10.0, m)
        elif kind == "unit":
            v = rng.uniform(-0.99, 0.99, m)
        else:
            v = rng.uniform(-4.0, 4.0, m)
        if kind == "special" and m >= 8:
            v[:: max(m // 8, 1)][:6] = [0.0, -0.0, np.inf, -np.inf, np.nan, 1.0][: len(v[:: max(m // 8, 1)][:6])]
        return v

    if dtype == "half":
        return f32_to_solid_half(reals(n).astype(np.float32))
    if dtype == "float":
        return reals(n).astype(np.float32)
    if dtype == "double":
        return reals(n).astype(np.float64)
    if dtype == "chalf":
        out = np.zeros(n, dtype=dt.CHALF_NP)
        out["real"] = f32_to_solid_half(reals(n).astype(np.float32))
        out["imag"] = f32_to_solid_half(reals(n).astype(np.float32))
        return out
    if dtype == "cfloat":
        return (reals(n) + 1j * reals(n)).astype(np.complex64)
    if dtype == "cdouble":
        return (reals(n) + 1j * reals(n)).astype(np.complex128)
    raise KeyError(dtype)


# ----------------------------------------------------------------------------
# views over flat buffers
# ----------------------------------------------------------------------------
class View:
    """A tensor view: `size` elements per dimension, `strides` in bytes, starting
    `offset` bytes into a flat byte buffer of `nbytes`."""

    def __init__(self, dtype, size, strides, offset, nbytes):
        self.dtype, self.size, self.strides, self.offset, self.nbytes = dtype, list(size), list(strides), offset, nbytes

    @property
    def nelem(self):
        n = 1
        for s in self.size:
            n *= s
        return n


def dense_view(dtype, size, offset_elems=0, pad_elems=0) -> View:
    """Column-major dense view (dimension 0 contiguous), optionally starting
    `offset_elems` elements into the buffer and with `pad_elems` extra elements per column."""
    es = dt.SIZE[dtype]
    strides, step = [], es
    for i, s in enumerate(size):
        strides.append(step)
        step *= (s + (pad_elems if i == 0 else 0))
    total = step if size else es
    return View(dtype, size, strides, offset_elems * es, total + offset_elems * es + 64)


def fill_buffer(view: View, rng, kind="general") -> np.ndarray:
    """A host byte buffer for `view`, completely filled with valid elements of its type."""
    es = dt.SIZE[view.dtype]
    n = view.nbytes // es
    vals = random_values(view.dtype, n + 1, rng, kind)
    buf = np.zeros(view.nbytes, dtype=np.uint8)
    head = view.offset % es              # keeps elements of unaligned views valid too
    raw = vals.view(np.uint8)
    m = min(len(raw), view.nbytes - head)
    buf[head: head + m] = raw[:m]
    return buf


def gather(buf: np.ndarray, view: View) -> np.ndarray:
    """Elements of the view in column-major order, as the numpy carrier type."""
    es = dt.SIZE[view.dtype]
    idx = np.zeros(1, dtype=np.int64)
    for s, st in zip(view.size, view.strides):          # dimension 0 varies fastest
        idx = (np.arange(s, dtype=np.int64)[:, None] * st + idx[None, :]).reshape(-1)
    bytes_idx = (idx[:, None] + view.offset + np.arange(es)[None, :]).reshape(-1)
    return buf[bytes_idx].view(dt.NUMPY[view.dtype]) if len(idx) else np.zeros(0, dtype=dt.NUMPY[view.dtype])


class Device:
    """Device mirror of host byte buffers (torch only allocates and copies)."""

    def __init__(self):
        import torch
        self.torch = torch

    def upload(self, buf: np.ndarray):
        t = self.torch.from_numpy(np.ascontiguousarray(buf)).cuda()
        return t

    def empty(self, nbytes: int):
        return self.torch.zeros(max(nbytes, 16), dtype=self.torch.uint8, device="cuda")

    def download(self, t) -> np.ndarray:
        self.torch.cuda.synchronize()
        return t.cpu().numpy()

    @property
    def stream(self):
        return self.torch.cuda.current_stream().cuda_stream


# ----------------------------------------------------------------------------
# comparison
# ----------------------------------------------------------------------------
def as_float_components(arr: np.ndarray, dtype: str) -> np.ndarray:
    """Real components of a floating-point typed array as float64 (half decoded)."""
    if dtype == "half":
        return arr.view(np.float16).astype(np.float64)
    if dtype == "chalf":
        return arr.view(np.uint16).view(np.float16).astype(np.float64)
    if dtype == "cfloat":
        return arr.view(np.float32).astype(np.float64)
    if dtype == "cdouble":
        return arr.view(np.float64)
    return arr.astype(np.float64)


def ulp_distance(a: np.ndarray, b: np.ndarray, dtype: str) -> np.ndarray:
    """Distance in units in the last place between two arrays of a floating type
    (0 where both are NaN; huge where exactly one is)."""
    comp = {"half": np.float16, "chalf": np.float16, "float": np.float32, "cfloat": np.float32,
            "double": np.float64, "cdouble": np.float64}[dtype]
    ibits = {np.float16: np.int16, np.float32: np.int32, np.float64: np.int64}[comp]
    fa = np.ascontiguousarray(a).view(np.uint8).view(comp)
    fb = np.ascontiguousarray(b).view(np.uint8).view(comp)
    ia = fa.view(ibits).astype(np.int64)
    ib = fb.view(ibits).astype(np.int64)
    sign = np.int64(np.iinfo(ibits).min)
    ia = np.where(ia < 0, sign - ia, ia)          # map to a monotone integer line
    ib = np.where(ib < 0, sign - ib, ib)
    d = np.abs(ia - ib)
    both_nan = np.isnan(fa) & np.isnan(fb)
    one_nan = np.isnan(fa) ^ np.isnan(fb)
    d = np.where(both_nan, 0, d)
    d = np.where(one_nan, np.int64(1) << 40, d)
    return d


def assert_same(got: np.ndarray, want: np.ndarray, dtype: str, ulp: int = 0, what: str = ""):
    """Bit-exact for integer and bool types; for floating types equal bits, or both NaN,
    or within `ulp` units in the last place."""
    assert got.shape == want.shape, what
    if dtype in dt.GROUPS["integer_bool"]:
        if ulp == 0:
            bad = np.nonzero(got != want)[0]
        else:                                        # integer results of functions evaluated in double
            bad = np.nonzero(np.abs(got.astype(np.float64) - want.astype(np.float64)) > ulp)[0]
        assert bad.size == 0, "%s: %d mismatches, first at %d: got %r want %r" % (
            what, bad.size, bad[0], got[bad[0]], want[bad[0]])
        return
    d = ulp_distance(got, want, dtype)
    bad = np.nonzero(d > ulp)[0]
    assert bad.size == 0, "%s: %d elements beyond %d ulp (max %d), first component %d: got %r want %r" % (
        what, bad.size, ulp, int(d.max()), bad[0],
        as_float_components(got, dtype)[bad[0]], as_float_components(want, dtype)[bad[0]])


# ----------------------------------------------------------------------------
# floating-point accumulations against a float64 evaluation
# ----------------------------------------------------------------------------
TIGHT_ACCUM = {"sum", "sum_nan", "sum_abs", "sum_abs_nan", "norm2", "norm2_nan"}


def as_values(arr: np.ndarray, dtype: str) -> np.ndarray:
    """Elements as float64 (real types, integers included) or complex128."""
    if dtype in dt.COMPLEX:
        c = as_float_components(arr, dtype).reshape(-1, 2)
        return c[:, 0] + 1j * c[:, 1]
    return as_float_components(arr, dtype).reshape(-1)


def f64_accumulate(op: str, x: np.ndarray, axis=None):
    """(value, scale) of sum / sum_abs / norm2 (and their NaN-skipping forms on real data) evaluated in float64.
    `scale` is what the rounding error of an accumulation is proportional to: the sum of magnitudes for sums,
    the value itself for norm2."""
    base = op[:-4] if op.endswith("_nan") else op
    if op.endswith("_nan"):
        x = np.where(np.isnan(x), 0, x)
    with np.errstate(invalid="ignore", over="ignore"):
        if base == "sum":
            if np.iscomplexobj(x):
                return x.sum(axis=axis), np.abs(x.real).sum(axis=axis) + np.abs(x.imag).sum(axis=axis)
            return x.sum(axis=axis), np.abs(x).sum(axis=axis)
        if base == "sum_abs":
            v = np.abs(x).sum(axis=axis)
            return v, v
        if base == "norm2":
            v = np.sqrt((x.real ** 2 + x.imag ** 2).sum(axis=axis)) if np.iscomplexobj(x) else np.sqrt((x * x).sum(axis=axis))
            return v, v
    raise KeyError(op)


def accumulation_bound(n: int, rdtype: str, scale):
    """Rounding-error bound of an n-term accumulation done as short sequential chains joined by a tree, in the
    accumulator type of `rdtype`: (4 log2 n + 4) u scale with u = 2^-24 (float, and half which accumulates in
    float) or 2^-53 (double).  (assert_accumulation adds one unit of the stored result for the half types.)

    Why this bound can fail where 1e-5 sqrt(n) sum|x| cannot: take values of typical magnitude m with random
    signs and drop k = max(1, n/100) of them.  The sum moves by about m sqrt(k); the bound is
    (4 log2 n + 4) 2^-24 n m.  n = 7: 1 m against 6e-6 m; n = 1000: 3.2 m against 2.6e-3 m; n = 70001:
    26 m against 0.29 m; n = 2^24: 410 m against 100 m; n = 2^26: 819 m against 432 m.  The old bound at
    n = 70001 is 1e-5 * 265 * 70001 m = 185 m, above the shift.  For sums of one sign (sum_abs, norm2, sums of
    squares) dropping 1 % moves the value by 1 % against a bound of 6e-6 at n = 2^26."""
    u = 2.0 ** -53 if rdtype in ("double", "cdouble") else 2.0 ** -24
    return (4 * np.log2(max(int(n), 2)) + 4) * u * np.asarray(scale, dtype=np.float64)


def assert_accumulation(got, truth, n, rdtype, scale, what):
    """|got - truth| <= accumulation_bound component-wise; equal infinities and NaN on both sides pass."""
    g = np.asarray(got)
    t = np.asarray(truth)
    if np.iscomplexobj(t) or np.iscomplexobj(g):
        g = np.stack([np.real(g), np.imag(g)], -1).astype(np.float64)
        t = np.stack([np.real(t), np.imag(t)], -1).astype(np.float64)
        scale = np.asarray(scale, dtype=np.float64)[..., None]
    bound = accumulation_bound(n, rdtype, scale) + 1e-300
    if rdtype in ("half", "chalf"):
        bound = bound + np.abs(t) * 2.0 ** -10
    with np.errstate(invalid="ignore"):
        ok = (np.isnan(g) & np.isnan(t)) | (np.isinf(g) & np.isinf(t) & (np.sign(g) == np.sign(t))) | (np.abs(g - t) <= bound)
        # a float64 evaluation that is finite where the narrower result type overflowed says nothing (beyond 65504
        # the reference's float -> half conversion gives infinities and, up to 131072, NaN patterns)
        limit = 65000.0 if rdtype in ("half", "chalf") else (3e38 if rdtype in ("float", "cfloat") else 1e308)
        ok |= ~np.isfinite(g) & (np.abs(t) > limit)
    assert np.all(ok), "%s: got %r, float64 evaluation %r, bound %r" % (what, g[~ok][:4], t[~ok][:4], np.broadcast_to(bound, g.shape)[~ok][:4])
