"""Parity of the elementwise entry points (unary, binary, fill) with the reference's
Solid CPU library on the same seeded buffers, through the C-ABI, over contiguous,
offset, padded, transposed, broadcast, reversed, scalar and in-place layouts.

Tolerances: bit-exact for bool/integer results and for IEEE operations (add,
subtract, multiply, divide, sqrt, min/max, rounding, sign, conj, ...); at most
2 ulp for the transcendental functions named by the benchmark configurations
(exp, log, sin and relatives on real types) and 4 ulp for the remaining
library functions, whose GPU and glibc implementations are different programs
(tests/test_gpu_ulp.py measures each side against the true value: both stay
within 1-3.5 ulp of it and within 3 ulp of each other).
"""
import zlib

import numpy as np
import pytest

import util
from solid_b200 import dtypes as dt
from solid_b200 import oplist as ol

pytestmark = pytest.mark.gpu

EXACT_UNARY = {"negative", "conj", "reciprocal", "bitwise_not", "logical_not", "sqrt", "square", "fabs", "sign",
               "ceil", "floor", "trunc", "round", "isinf", "isnan", "isfinite", "isposinf", "isneginf", "absolute"}
ULP2_UNARY = {"sin", "cos", "exp", "log", "exp2", "log2", "log10", "expm1", "log1p", "arctan"}
DOMAIN = {"arcsin": "unit", "arccos": "unit", "arctanh": "unit", "arccosh": "positive",
          "log": "positive", "log2": "positive", "log10": "positive", "log1p": "positive", "sqrt": "positive"}


def unary_tolerance(op, dtype):
    if dtype in dt.GROUPS["integer_bool"]:
        return 0 if op in EXACT_UNARY else 1          # integer results of double-precision library functions
    if dtype in dt.COMPLEX:
        if op in {"negative", "conj", "square", "ceil", "floor", "trunc", "round", "isinf", "isnan", "isfinite"}:
            return 0
        if op in {"absolute", "fabs", "reciprocal", "sign"}:
            return 2                                   # one hypot / division
        if op in {"tan", "tanh"}:
            return -4096                               # quotients whose denominator cancels near the poles
        return -64                                     # compositions of several library functions: see below
    if op in EXACT_UNARY:
        return 0
    return 2 if op in ULP2_UNARY else 4          # measured distance between the two sides: at most 3 (test_gpu_ulp.py)


def assert_complex_close(got, want, dtype, units, what):
    """Complex elementary functions are formulas over several real library calls with
    cancellation between them, so the error is measured against the magnitude of the complex
    result: |got - want| <= units * eps * max(1, |want|) per component."""
    eps = {"chalf": 2.0 ** -10, "cfloat": 2.0 ** -23, "cdouble": 2.0 ** -52}[dtype]
    g = util.as_float_components(got, dtype).reshape(-1, 2)
    w = util.as_float_components(want, dtype).reshape(-1, 2)
    mag = np.maximum(1.0, np.hypot(w[:, 0], w[:, 1]))[:, None]
    with np.errstate(invalid="ignore"):
        ok = (np.isnan(g) & np.isnan(w)) | (g == w) | (np.abs(g - w) <= units * eps * mag)
    bad = np.nonzero(~ok.all(axis=1))[0]
    assert bad.size == 0, "%s: %d elements off, first %d: got %r want %r" % (what, bad.size, bad[0], g[bad[0]], w[bad[0]])


def layouts(dtype, out_dtype=None):
    """(name, size, view of operand 1, view of result) cases."""
    od = out_dtype or dtype
    es, eo = dt.SIZE[dtype], dt.SIZE[od]
    cases = []
    for n in (0, 1, 7, 1000, 4099):
        cases.append(("contig%d" % n, [n], util.dense_view(dtype, [n]), util.dense_view(od, [n])))
    cases.append(("offset", [1003], util.dense_view(dtype, [1003], offset_elems=1), util.dense_view(od, [1003], offset_elems=3)))
    cases.append(("padded", [32, 9], util.dense_view(dtype, [32, 9], pad_elems=16), util.dense_view(od, [32, 9], pad_elems=16)))
    cases.append(("padded_odd", [13, 7], util.dense_view(dtype, [13, 7], pad_elems=3), util.dense_view(od, [13, 7])))
    v = util.dense_view(dtype, [11, 37]); vt = util.View(dtype, [37, 11], [v.strides[1], v.strides[0]], 0, v.nbytes)
    cases.append(("transposed", [37, 11], vt, util.dense_view(od, [37, 11])))
    vb = util.View(dtype, [40, 6], [0, es], 0, 6 * es + 64)
    cases.append(("row_broadcast", [40, 6], vb, util.dense_view(od, [40, 6])))
    vs = util.View(dtype, [50, 3], [0, 0], 0, 64)
    cases.append(("scalar_broadcast", [50, 3], vs, util.dense_view(od, [50, 3])))
    v3 = util.dense_view(dtype, [5, 6, 7])
    vr = util.View(dtype, [5, 6, 7], [v3.strides[0], -v3.strides[1], v3.strides[2]], 5 * v3.strides[1], v3.nbytes)
    cases.append(("reversed_dim", [5, 6, 7], vr, util.dense_view(od, [5, 6, 7])))
    cases.append(("zero_dim", [], util.dense_view(dtype, []), util.dense_view(od, [])))
    return cases


def out_type_unary(op, dtype):
    if op in ("isinf", "isnan", "isfinite", "isposinf", "isneginf"):
        return "bool"
    if op == "absolute":
        return dt.elem_type(dtype)
    return dtype


@pytest.mark.parametrize("op", sorted(ol.UNARY_OPS))
def test_unary_matches_reference(op, gpu, cpu):
    dev = util.Device()
    for dtype in dt.GROUPS[ol.UNARY_OPS[op]]:
        if op == "arctanh" and dtype in dt.COMPLEX:
            continue          # the reference never writes the real part (unary_ops.h:472-474)
        od = out_type_unary(op, dtype)
        kind = DOMAIN.get(op, "special" if op in EXACT_UNARY else "general")
        if dtype in dt.GROUPS["integer_bool"] and op not in EXACT_UNARY:
            kind = "small" if op in ("exp", "exp2", "exp10", "expm1", "sinh", "cosh") else kind
            if op in ("exp10",):
                kind = "unit"
        rng = np.random.default_rng(zlib.crc32(("%s %s" % (op, dtype)).encode()))
        for name, size, vin, vout in layouts(dtype, od):
            src = util.fill_buffer(vin, rng, kind)
            dst0 = util.fill_buffer(vout, rng, "general")
            want = dst0.copy()
            cpu.unary(op, dtype, size, vin.strides, src.ctypes.data + vin.offset, vout.strides, want.ctypes.data + vout.offset)
            dsrc, ddst = dev.upload(src), dev.upload(dst0)
            gpu.unary(op, dtype, size, vin.strides, dsrc.data_ptr() + vin.offset, vout.strides,
                      ddst.data_ptr() + vout.offset, dev.stream)
            got = dev.download(ddst)
            what = "%s_%s %s" % (op, dtype, name)
            # bytes outside the view must be untouched; inside compare with the op's tolerance
            g, w = util.gather(got, vout), util.gather(want, vout)
            tol = unary_tolerance(op, dtype)
            if op == "cbrt" and dtype == "cdouble":
                # the oracle's complex cube root goes through its single-precision pow (mathfn.cuh)
                assert_complex_close(g.astype(np.complex64), w.astype(np.complex64), "cfloat", 64, what)
            elif tol < 0:
                assert_complex_close(g, w, od, -tol, what)
            else:
                util.assert_same(g, w, od, tol, what)
            mask = np.ones(len(got), dtype=bool)
            if vout.nelem:
                idx = np.zeros(1, dtype=np.int64)
                for s, st in zip(vout.size, vout.strides):
                    idx = (np.arange(s, dtype=np.int64)[:, None] * st + idx[None, :]).reshape(-1)
                mask[(idx[:, None] + vout.offset + np.arange(dt.SIZE[od])[None, :]).reshape(-1)] = False
            assert np.array_equal(got[mask], dst0[mask]), what + ": wrote outside the destination view"


def test_unary_in_place(gpu, cpu):
    dev = util.Device()
    rng = np.random.default_rng(5)
    for dtype, op in (("float", "sqrt"), ("int32", "negative"), ("cdouble", "conj"), ("half", "square")):
        v = util.dense_view(dtype, [777])
        src = util.fill_buffer(v, rng, "positive")
        want = src.copy()
        cpu.unary(op, dtype, v.size, v.strides, want.ctypes.data, v.strides, want.ctypes.data)
        d = dev.upload(src)
        gpu.unary(op, dtype, v.size, v.strides, d.data_ptr(), v.strides, d.data_ptr(), dev.stream)
        util.assert_same(util.gather(dev.download(d), v), util.gather(want, v), dtype, 0, "%s in place" % op)


# ---------------------------------------------------------------------------
EXACT_BINARY = set(ol.BINARY_OPS) - {"power", "fmod"}


def second_type(op, dtype):
    if op in ("bitshift_left", "bitshift_right"):
        return "int8"
    if op == "power" and dtype in dt.GROUPS["integer_bool"]:
        return "int16"
    return dtype


def out_type_binary(op, dtype):
    return "bool" if op in ol.COMPARE_OPS else dtype


def second_values(op, dtype, n, rng):
    if op in ("bitshift_left", "bitshift_right"):
        return rng.integers(-3, min(8, 8 * dt.SIZE[dtype]), n).astype(np.int8)
    if op == "power" and dtype in dt.GROUPS["integer_bool"]:
        return rng.integers(-2, 5, n).astype(np.int16)
    return None


@pytest.mark.parametrize("op", sorted(ol.BINARY_OPS))
def test_binary_matches_reference(op, gpu, cpu):
    dev = util.Device()
    for dtype in dt.GROUPS[ol.BINARY_OPS[op]]:
        t2, od = second_type(op, dtype), out_type_binary(op, dtype)
        rng = np.random.default_rng(zlib.crc32(("%s %s b" % (op, dtype)).encode()))
        kind = "special" if (op in EXACT_BINARY and dtype in dt.GROUPS["float"]) else "general"
        if dtype in dt.GROUPS["integer"] and op in ("multiply", "power"):
            kind = "small"
        tol = 0
        if op == "power" and dtype in dt.GROUPS["float"]:
            tol, kind = 64, "positive"                     # single-precision pow inside (see mathfn.cuh)
        if op == "fmod" and dtype in dt.REAL:
            tol = 0
        if dtype in dt.COMPLEX and op in ("divide", "true_divide"):
            tol = 0
        base_cases = layouts(dtype, od)
        for i, (name, size, v1, vout) in enumerate(base_cases):
            # second operand: dense, or a broadcast row/scalar for some cases
            if name == "padded":
                v2 = util.View(t2, size, [0, dt.SIZE[t2]], 0, size[1] * dt.SIZE[t2] + 64)
            elif name == "contig1000":
                v2 = util.View(t2, size, [0], 0, 64)
            else:
                v2 = util.dense_view(t2, size)
            a = util.fill_buffer(v1, rng, kind)
            b = util.fill_buffer(v2, rng, kind)
            sv = second_values(op, dtype, v2.nbytes // dt.SIZE[t2], rng)
            if sv is not None:
                b = np.zeros(v2.nbytes, dtype=np.uint8); raw = sv.view(np.uint8); b[: len(raw)] = raw[: len(b)]
            dst0 = util.fill_buffer(vout, rng, "general")
            want = dst0.copy()
            cpu.binary(op, dtype, size, v1.strides, a.ctypes.data + v1.offset, v2.strides, b.ctypes.data + v2.offset,
                       vout.strides, want.ctypes.data + vout.offset)
            da, db, dd = dev.upload(a), dev.upload(b), dev.upload(dst0)
            gpu.binary(op, dtype, size, v1.strides, da.data_ptr() + v1.offset, v2.strides, db.data_ptr() + v2.offset,
                       vout.strides, dd.data_ptr() + vout.offset, dev.stream)
            got = dev.download(dd)
            g, w = util.gather(got, vout), util.gather(want, vout)
            if op == "power" and dtype in dt.COMPLEX:
                # exp(y*log(x)): the error of the logarithm is multiplied by |y log x|
                gd = g.astype(np.complex64) if dtype == "cdouble" else g
                wd = w.astype(np.complex64) if dtype == "cdouble" else w
                assert_complex_close(gd, wd, "cfloat" if dtype == "cdouble" else dtype, 8192, "%s_%s %s" % (op, dtype, name))
            elif op == "power" and dtype in ("double", "cdouble"):
                # the oracle evaluates double pow in single precision (SOLID_DOUBLE_POW is powf), so
                # the comparison is made at single precision too
                cd = np.complex64 if dtype == "cdouble" else np.float32
                g, w = g.astype(cd), w.astype(cd)
                util.assert_same(g, w, "cfloat" if dtype == "cdouble" else "float", tol, "%s_%s %s" % (op, dtype, name))
            else:
                util.assert_same(g, w, od, tol, "%s_%s %s" % (op, dtype, name))


@pytest.mark.parametrize("dtype", dt.NAMES)
def test_fill_and_masked_fill(dtype, gpu, cpu):
    dev = util.Device()
    rng = np.random.default_rng(dt.INDEX[dtype])
    value = util.random_values(dtype, 1, rng).tobytes()
    for name, size, v, _ in layouts(dtype):
        if name in ("row_broadcast", "scalar_broadcast"):
            continue                                     # a destination cannot be a broadcast view
        buf = util.fill_buffer(v, rng)
        want = buf.copy()
        cpu.fill("fill", dtype, size, v.strides, want.ctypes.data + v.offset, value)
        d = dev.upload(buf)
        gpu.fill("fill", dtype, size, v.strides, d.data_ptr() + v.offset, value, dev.stream)
        assert np.array_equal(dev.download(d), want), "fill_%s %s" % (dtype, name)
        # masked fill
        vm = util.dense_view("bool", size)
        mask = util.fill_buffer(vm, rng)
        want = buf.copy()
        cpu.masked_fill(dtype, size, v.strides, want.ctypes.data + v.offset, vm.strides, mask.ctypes.data, value)
        d, dm = dev.upload(buf), dev.upload(mask)
        gpu.masked_fill(dtype, size, v.strides, d.data_ptr() + v.offset, vm.strides, dm.data_ptr(), value, dev.stream)
        assert np.array_equal(dev.download(d), want), "masked_fill_%s %s" % (dtype, name)
    if dtype in dt.GROUPS["float"]:
        v = util.dense_view(dtype, [999])
        buf = util.fill_buffer(v, rng, "special")
        want = buf.copy()
        cpu.fill("fill_nan", dtype, v.size, v.strides, want.ctypes.data, value)
        d = dev.upload(buf)
        gpu.fill("fill_nan", dtype, v.size, v.strides, d.data_ptr(), value, dev.stream)
        assert np.array_equal(dev.download(d), want), "fill_nan_%s" % dtype


@pytest.mark.parametrize("op", sorted(ol.SCALAR_OPS))
def test_scalar_operand_by_value_matches_broadcast_tensor(op, gpu, cpu):
    """solid_gpu_<op>_scalar_<type> takes the second operand by value; the oracle is the reference's tensor
    operation with that scalar as a stride-0 second operand (what Ocean's addScalar and relatives run).
    Bit-exact, including the in-place form (no destination given)."""
    dev = util.Device()
    for dtype in dt.GROUPS[ol.SCALAR_OPS[op]]:
        rng = np.random.default_rng(zlib.crc32(("%s %s s" % (op, dtype)).encode()))
        kind = "small" if (dtype in dt.GROUPS["integer"] and op == "multiply") else \
               ("special" if dtype in dt.GROUPS["float"] else "general")
        es = dt.SIZE[dtype]
        for name, size, v1, vout in layouts(dtype):
            if name in ("row_broadcast", "scalar_broadcast"):
                continue                                # a source that overlaps itself cannot be updated in place
            a = util.fill_buffer(v1, rng, kind)
            s = util.random_values(dtype, 1, rng, kind)
            sbuf = np.zeros(64, dtype=np.uint8); sbuf[:es] = s.view(np.uint8)[:es]
            zero = [0] * len(size)
            for in_place in (False, True):
                vo = v1 if in_place else vout
                dst0 = a.copy() if in_place else util.fill_buffer(vout, rng, "general")
                want = dst0.copy()
                src = want if in_place else a
                cpu.binary(op, dtype, size, v1.strides, src.ctypes.data + v1.offset, zero, sbuf.ctypes.data,
                           vo.strides, want.ctypes.data + vo.offset)
                da, dd = dev.upload(a), dev.upload(dst0)
                if in_place:
                    gpu.scalar_op(op, dtype, size, v1.strides, dd.data_ptr() + v1.offset, sbuf[:es].tobytes(), None, None, dev.stream)
                else:
                    gpu.scalar_op(op, dtype, size, v1.strides, da.data_ptr() + v1.offset, sbuf[:es].tobytes(),
                                  vo.strides, dd.data_ptr() + vo.offset, dev.stream)
                got = dev.download(dd)
                util.assert_same(util.gather(got, vo), util.gather(want, vo), dtype, 0,
                                 "%s_scalar_%s %s%s" % (op, dtype, name, " in place" if in_place else ""))


@pytest.mark.parametrize("op", sorted(ol.CHECKED_OPS))
def test_checked_unary_equals_function_plus_domain_reduction(op, gpu, cpu):
    """solid_gpu_<op>_checked_<type> = the unary function (compared with the tolerance of that function) and the
    domain test the reference runs as a separate global reduction: not all_ge(bound) / not all in [-1, 1] /
    not all (nonzero), computed here with the reference's own reductions on the same data."""
    dev = util.Device()
    bounds = {"sqrt": ("all_ge", 0.0), "log": ("all_ge", 0.0), "log2": ("all_ge", 0.0), "log10": ("all_ge", 0.0),
              "log1p": ("all_ge", -1.0), "arccosh": ("all_ge", 1.0)}
    for dtype in dt.GROUPS[ol.CHECKED_OPS[op]]:
        rng = np.random.default_rng(zlib.crc32(("%s %s c" % (op, dtype)).encode()))
        es = dt.SIZE[dtype]
        tol = unary_tolerance(op, dtype)
        for name, size, v1, vout in layouts(dtype):
            if name in ("row_broadcast", "scalar_broadcast"):
                continue
            for kind in ("inside", "outside", "nan"):
                inside_kind = {"arcsin": "unit", "arccos": "unit", "arctanh": "unit"}.get(op, "positive")
                a = util.fill_buffer(v1, rng, inside_kind)
                vals = util.gather(a, v1).copy()
                if op == "arccosh":
                    vals = (sn_half(vals, dtype, lambda f: f + 1.0))
                if vals.size and kind != "inside":
                    pos = int(rng.integers(0, vals.size))
                    bad = {"outside": {"arcsin": 1.5, "arccos": -1.5, "arctanh": 2.0, "arccosh": 0.5, "log1p": -1.5,
                                       "reciprocal": 0.0}.get(op, -0.25), "nan": float("nan")}[kind]
                    vals = sn_half(vals, dtype, lambda f: np.where(np.arange(f.size) == pos, bad, f))
                a = scatter_into(a, v1, vals)
                dst0 = util.fill_buffer(vout, rng, "general")
                want = dst0.copy()
                cpu.unary(op, dtype, size, v1.strides, a.ctypes.data + v1.offset, vout.strides, want.ctypes.data + vout.offset)
                if op in bounds:
                    red, b = bounds[op]
                    ok = cpu.reduce_all(red, dtype, size, v1.strides, a.ctypes.data + v1.offset,
                                        bounds=(scalar_of(b, dtype),))[0]
                elif op == "reciprocal":
                    ok = cpu.reduce_all("all", dtype, size, v1.strides, a.ctypes.data + v1.offset)[0]
                else:
                    ok = cpu.reduce_all("all_gele", dtype, size, v1.strides, a.ctypes.data + v1.offset,
                                        bounds=(scalar_of(-1.0, dtype), scalar_of(1.0, dtype)))[0]
                # the data does what the case says (a NaN fails none of the reference's comparisons)
                expect_ok = kind != "outside" or vals.size == 0
                assert bool(ok) == expect_ok, ("test data", op, dtype, name, kind)
                da, dd = dev.upload(a), dev.upload(dst0)
                flag = dev.empty(16)
                gpu.unary_checked(op, dtype, size, v1.strides, da.data_ptr() + v1.offset, vout.strides,
                                  dd.data_ptr() + vout.offset, flag.data_ptr(), dev.stream)
                got = dev.download(dd)
                what = "%s_checked_%s %s %s" % (op, dtype, name, kind)
                util.assert_same(util.gather(got, vout), util.gather(want, vout), dtype, tol, what)
                assert int(dev.download(flag)[:4].view(np.int32)[0]) == (0 if ok else 1), what


def sn_half(vals, dtype, fn):
    """Apply fn to the values as float64 and return them in the carrier of dtype (half through the oracle's rounding)."""
    from oracle import solid_numpy as sn
    if dtype == "half":
        f = sn.half_to_float(vals).astype(np.float64)
        return sn.float_to_half(np.asarray(fn(f), dtype=np.float32))
    return np.asarray(fn(vals.astype(np.float64))).astype(vals.dtype)


def scatter_into(buf, view, vals):
    """Write the elements of `vals` (logical column-major order of the view) back into a copy of the byte buffer."""
    out = buf.copy()
    es = dt.SIZE[view.dtype]
    raw = np.ascontiguousarray(vals).view(np.uint8).reshape(-1, es)
    idx = np.zeros(1, dtype=np.int64)
    for d in range(len(view.size) - 1, -1, -1):
        idx = (idx[:, None] + (np.arange(view.size[d], dtype=np.int64) * view.strides[d])[None, :]).reshape(-1)
    if raw.shape[0]:
        out[(view.offset + idx)[:, None] + np.arange(es)[None, :]] = raw
    return out


def scalar_of(value, dtype):
    from solid_b200 import ops
    return ops.scalar_bytes(value, dtype)
