"""Pins the numpy restatement (oracle/solid_numpy.py) to the reference:
(1) against the committed golden vectors, which the reference's Solid CPU library produced
    (tests/golden/make_golden.py), and
(2) against that library itself on fresh seeded inputs wherever oracle/_ref is present.
Exact operations must agree bit for bit; library functions within 2 ulp; floating sums within
the tolerance the parity tests use."""
import zlib
from pathlib import Path

import numpy as np
import pytest

import util
from oracle import solid_numpy as sn
from solid_b200 import dtypes as dt, oplist as ol

GOLDEN = Path(__file__).resolve().parent / "golden" / "solid_cpu_golden.npz"
LIBM_UNARY = {"exp", "log", "sin"}
INEXACT_BINARY = {"power", "fmod"}
FLOAT_ACCUM = {"sum", "prod", "sum_abs", "norm2"}


@pytest.fixture(scope="module")
def golden():
    return np.load(GOLDEN)


def keys(golden, family):
    return sorted({tuple(k.split("/")[1:3]) for k in golden.files if k.startswith(family + "/")})


def test_golden_unary(golden):
    checked = 0
    for op, dtype in keys(golden, "unary"):
        if dtype in dt.COMPLEX and op not in ("negative", "conj", "square", "absolute", "fabs", "ceil", "floor", "trunc",
                                              "isinf", "isnan", "isfinite", "exp", "log", "reciprocal"):
            continue
        x, want = golden["unary/%s/%s/in" % (op, dtype)], golden["unary/%s/%s/out" % (op, dtype)]
        got = sn.unary(op, dtype, x)
        od = "bool" if op.startswith("is") else (dt.elem_type(dtype) if op == "absolute" else dtype)
        tol = 0
        if op in LIBM_UNARY:
            tol = 1 if dtype in dt.GROUPS["integer"] else 2
        if dtype in dt.COMPLEX and op in ("absolute", "fabs", "exp", "log", "reciprocal"):
            tol = 4
        util.assert_same(np.asarray(got), want, od, tol, "unary %s %s" % (op, dtype))
        checked += 1
    assert checked > 200


def test_golden_binary(golden):
    checked = 0
    for op, dtype in keys(golden, "binary"):
        if dtype in dt.COMPLEX and op == "power":
            continue
        x, y = golden["binary/%s/%s/in1" % (op, dtype)], golden["binary/%s/%s/in2" % (op, dtype)]
        want = golden["binary/%s/%s/out" % (op, dtype)]
        got = sn.binary(op, dtype, x, y)
        od = "bool" if op in ol.COMPARE_OPS else dtype
        tol = 0
        if op == "power" and dtype in dt.REAL:
            g, w = sn.to_work(dtype, got).astype(np.float32), sn.to_work(dtype, want).astype(np.float32)
            util.assert_same(g, w, "float", 16, "binary power %s" % dtype)
        else:
            util.assert_same(np.asarray(got), want, od, tol, "binary %s %s" % (op, dtype))
        checked += 1
    assert checked > 300


def test_golden_copy(golden):
    for src, dst in keys(golden, "copy"):
        x = golden["copy/%s/%s/in" % (src, dst)]
        assert sn.convert(src, dst, x).tobytes() == golden["copy/%s/%s/out" % (src, dst)].tobytes(), (src, dst)
        # byteswap_copy treats the stored bytes as reversed
        xs = golden["copy/%s/%s/in_swapped" % (src, dst)]
        assert xs.tobytes() == sn.byteswap(src, x).tobytes(), (src, "byteswap")
        assert sn.byteswap_convert(src, dst, xs).tobytes() == golden["copy/%s/%s/out_swapped_source" % (src, dst)].tobytes(), (src, dst)


def test_golden_reduce(golden):
    for op, dtype in keys(golden, "reduce"):
        x, want = golden["reduce/%s/%s/in" % (op, dtype)], golden["reduce/%s/%s/out" % (op, dtype)]
        got = np.asarray(sn.reduce_all(op, dtype, x)).reshape(1)
        rtype = ol.reduce_result_type(op, dtype)
        if op in FLOAT_ACCUM and rtype in dt.GROUPS["float"]:
            g, w = util.as_float_components(got.astype(want.dtype), rtype), util.as_float_components(want, rtype)
            eps = {"half": 2e-3, "chalf": 2e-3, "float": 1e-5, "cfloat": 1e-5}.get(rtype, 1e-12)
            scale = max(float(np.abs(util.as_float_components(x, dtype)).sum()), float(np.abs(w).max()), 1e-30)
            assert np.all(np.abs(g - w) <= eps * np.sqrt(len(x)) * scale), (op, dtype, g, w)
        else:
            util.assert_same(got.astype(want.dtype), want, rtype, 2 if (dtype in dt.COMPLEX and op.endswith("_abs")) else 0,
                             "reduce %s %s" % (op, dtype))


def test_half_rounding_known_answers():
    """The reference's float -> half conversion (solid/src/base/generic/half.c:101-149) on the cases
    where it differs from IEEE round-to-nearest-even."""
    f = np.array([1.0 + 2.0 ** -11, 1.0 + 3 * 2.0 ** -11, 2.0 ** -15, 2.0 ** -16, -2.0 ** -20, 65520.0, 70000.0,
                  131072.0, np.nan, -0.0], dtype=np.float32)
    want = np.array([0x3C01,      # tie rounds AWAY from zero (IEEE would give 0x3C00)
                     0x3C02,      # tie away again (IEEE: 0x3C02 as well)
                     0x0000,      # exponent 112 is re-biased to 0 with an empty mantissa
                     0x0000, 0x0000,  # below 2^-15: +0, sign dropped
                     0x7C00,      # rounds up into the infinity pattern
                     0x7C46,      # exponent 143 is encoded "as is": a NaN pattern (0x45 rounded up)
                     0x7C00,      # >= 2^17: infinity
                     0x7F00,      # NaN
                     0x0000], dtype=np.uint16)
    assert np.array_equal(sn.float_to_half(f), want), [hex(v) for v in sn.float_to_half(f)]
    h = np.array([0x8000, 0x0001, 0x7C00, 0xFC00, 0x3C00], dtype=np.uint16)
    got = sn.half_to_float(h)
    assert got[0] == 0 and not np.signbit(got[0])              # -0 decodes to +0
    assert got[1] == np.float32(2.0 ** -24) and np.isposinf(got[2]) and np.isneginf(got[3]) and got[4] == 1.0


def test_restatement_matches_reference_library(cpu):
    """Fresh inputs through both checkers (needs oracle/_ref)."""
    n = 257
    for dtype in dt.NAMES:
        rng = np.random.default_rng(zlib.crc32(dtype.encode()))
        x, y = util.random_values(dtype, n, rng), util.random_values(dtype, n, rng)
        for op in ("add", "subtract", "multiply", "min", "max", "eq", "lt"):
            od = "bool" if op in ol.COMPARE_OPS else dtype
            z = np.zeros(n, dtype=dt.NUMPY[od])
            cpu.binary(op, dtype, [n], [dt.SIZE[dtype]], x.ctypes.data, [dt.SIZE[dtype]], y.ctypes.data, [dt.SIZE[od]], z.ctypes.data)
            util.assert_same(np.asarray(sn.binary(op, dtype, x, y)), z, od, 0, "%s %s" % (op, dtype))
        if dtype in dt.GROUPS["all_nocomplex"] and dtype != "bool":
            safe = np.where(sn.to_work(dtype, y) == 0, x, y) if dtype not in dt.REAL else y
            for op in ("divide", "true_divide", "floor_divide", "mod"):
                z = np.zeros(n, dtype=dt.NUMPY[dtype])
                cpu.binary(op, dtype, [n], [dt.SIZE[dtype]], x.ctypes.data, [dt.SIZE[dtype]], y.ctypes.data, [dt.SIZE[dtype]], z.ctypes.data)
                util.assert_same(np.asarray(sn.binary(op, dtype, x, y)), z, dtype, 0, "%s %s" % (op, dtype))
        for dst in dt.NAMES:
            src_vals = util.random_values(dtype, n, rng, "positive" if (dst in dt.UINT or dst == "bool") else "general")
            out = np.zeros(n, dtype=dt.NUMPY[dst])
            cpu.copy(dtype, dst, [n], [dt.SIZE[dtype]], src_vals.ctypes.data, [n], [dt.SIZE[dst]], out.ctypes.data)
            assert sn.convert(dtype, dst, src_vals).tobytes() == out.tobytes(), (dtype, dst)
        for op in ("any", "all", "nnz", "maximum", "minimum"):
            rtype = ol.reduce_result_type(op, dtype)
            raw = cpu.reduce_all(op, dtype, [n], [dt.SIZE[dtype]], x.ctypes.data)
            want = np.frombuffer(raw[: dt.SIZE[rtype]], dtype=dt.NUMPY[rtype])
            util.assert_same(np.asarray(sn.reduce_all(op, dtype, x)).reshape(1).astype(want.dtype), want, rtype, 0, "%s %s" % (op, dtype))


def test_fused_sequences_match_reference_library(cpu):
    """axpy and the mixed multiply-add are defined as the reference's kernel sequences."""
    n = 513
    rng = np.random.default_rng(77)
    for dtype in dt.REAL:
        x, y = util.random_values(dtype, n, rng), util.random_values(dtype, n, rng)
        a = util.random_values(dtype, 1, rng)
        es = dt.SIZE[dtype]
        t, z = np.zeros(n, dtype=dt.NUMPY[dtype]), np.zeros(n, dtype=dt.NUMPY[dtype])
        cpu.binary("multiply", dtype, [n], [es], x.ctypes.data, [0], a.ctypes.data, [es], t.ctypes.data)
        cpu.binary("add", dtype, [n], [es], t.ctypes.data, [es], y.ctypes.data, [es], z.ctypes.data)
        aval = sn.to_work(dtype, a)[0]
        assert np.array_equal(sn.axpy(dtype, aval, x, y), z), dtype
    # C(float) = A(double) * B(int32, bytes reversed) + r(float)
    A = rng.uniform(-1, 1, n); B = rng.integers(-1000, 1001, n).astype(np.int32); r = rng.uniform(-1, 1, n).astype(np.float32)
    Bs = B.astype(">i4").view(np.int32)
    Bd, rd, P, S, Cw = (np.zeros(n) for _ in range(5))
    Cf = np.zeros(n, dtype=np.float32)
    cpu.copy("int32", "double", [n], [4], Bs.ctypes.data, [n], [8], Bd.ctypes.data, variant="byteswap_copy")
    cpu.copy("float", "double", [n], [4], r.ctypes.data, [n], [8], rd.ctypes.data)
    cpu.binary("multiply", "double", [n], [8], A.ctypes.data, [8], Bd.ctypes.data, [8], P.ctypes.data)
    cpu.binary("add", "double", [n], [8], P.ctypes.data, [8], rd.ctypes.data, [8], S.ctypes.data)
    cpu.copy("double", "float", [n], [8], S.ctypes.data, [n], [4], Cf.ctypes.data)
    got = sn.mixed_multiply_add("double", "float", A, "double", Bs, "int32", r, "float", swapped=(False, True, False))
    assert np.array_equal(got, Cf)


def test_ranges_and_indexed_access_match_reference_library(cpu):
    """The numpy restatements of steps_*, get/set/fill_index, add_if_negative and index_to_offset against the
    compiled reference (needs oracle/_ref)."""
    rng = np.random.default_rng(5)
    n = 300
    for dtype in dt.NAMES:
        es = dt.SIZE[dtype]
        kinds = [("int64", 7, 3), ("int64", -5, 2), ("double", 0.25, 0.5), ("double", 100.0, -0.375)]
        if dtype in dt.COMPLEX:
            kinds.append(("cdouble", 1 - 2j, 0.5 + 0.25j))
        for kind, off, step in kinds:
            if kind == "double" and step < 0 and (dtype in dt.UINT or dtype == "bool"):
                continue                                    # negative double -> unsigned: undefined in C, not restated
            if kind == "int64" and off < 0 and dtype == "half":
                pass                                        # 2^64-ish values: float_to_half saturates to inf the same way
            buf = np.zeros(n * es, dtype=np.uint8)
            cpu.steps(kind, dtype, [n], [es], buf.ctypes.data, off, step)
            got = sn.steps(kind, dtype, n, off, step)
            assert got.tobytes() == buf.tobytes(), (kind, dtype, off, step)
        # gather / scatter / fill through a table on dimension 0 and a stride on dimension 1 (column-major 40 x 30)
        src = rng.integers(0, 256, 40 * 30 * es).astype(np.uint8)
        tab = (rng.permutation(40)[:17].astype(np.int64)) * es
        sel = np.zeros(17 * 30 * es, dtype=np.uint8)
        cpu.index2("get_index", dtype, [17, 30], [tab.ctypes.data, None], [0, 40 * es], src.ctypes.data, [es, 17 * es], sel.ctypes.data)
        assert np.array_equal(sn.get_index(src, es, [17, 30], [tab, None], [0, 40 * es]).reshape(-1), sel), dtype
        dst = src.copy(); want = src.copy()
        vals = rng.integers(0, 256, 17 * 30 * es).astype(np.uint8)
        cpu.index2("set_index", dtype, [17, 30], [tab.ctypes.data, None], [0, 40 * es], want.ctypes.data, [es, 17 * es], vals.ctypes.data)
        sn.set_index(dst, es, [17, 30], [tab, None], [0, 40 * es], vals.reshape(-1, es))
        assert np.array_equal(dst, want), dtype
        value = rng.integers(0, 256, es).astype(np.uint8)
        dst = src.copy(); want = src.copy()
        cpu.fill_index(dtype, [17, 30], [tab.ctypes.data, None], [0, 40 * es], want.ctypes.data, value.tobytes())
        sn.set_index(dst, es, [17, 30], [tab, None], [0, 40 * es], np.broadcast_to(value, (17 * 30, es)))
        assert np.array_equal(dst, want), dtype
    for dtype in dt.SINT:
        x = rng.integers(-60, 60, 500).astype(dt.NUMPY[dtype])
        want = x.copy()
        cpu.add_if_negative(dtype, [500], [dt.SIZE[dtype]], want.ctypes.data, np.array([60], dtype=dt.NUMPY[dtype]).tobytes())
        assert np.array_equal(sn.add_if_negative(x, 60), want), dtype
    for dtype in dt.UINT + dt.SINT:
        idx = np.asfortranarray(rng.integers(0, 100, (3, 200)).astype(dt.NUMPY[dtype]))
        strides = [8, -640, 5120]
        es = dt.SIZE[dtype]
        out = np.zeros(200, dtype=np.int64)
        cpu.index_to_offset(dtype, strides, es, 200, 3 * es, idx.ctypes.data, 8, out.ctypes.data)
        assert np.array_equal(sn.index_to_offset(idx, strides), out), dtype


def test_golden_steps_and_gemm(golden):
    """Ranges and integer / bool matrix products of the numpy restatement against the committed outputs of the
    reference's Solid CPU library."""
    checked = 0
    for key in sorted(k for k in golden.files if k.startswith("steps/") and k.endswith("/out")):
        _, kind, dtype, j, _ = key.split("/")
        off, step = golden["steps/%s/%s/%s/param" % (kind, dtype, j)]
        if kind == "int64":
            off, step = int(off.real), int(step.real)
        elif kind == "double":
            off, step = float(off.real), float(step.real)
        want = golden[key]
        n = want.size // dt.SIZE[dtype]
        assert sn.steps(kind, dtype, n, off, step).tobytes() == want.tobytes(), key
        checked += 1
    for key in sorted(k for k in golden.files if k.startswith("gemm/") and k.endswith("/out")):
        _, trans, dtype, _ = key.split("/")
        base = key[: -len("/out")]
        m, n, k, lda, ldb, ldc, alpha, beta = (int(v) for v in golden[base + "/param"])
        got = sn.gemm(dtype, trans[0], trans[1], m, n, k, alpha, golden[base + "/A"], lda, golden[base + "/B"], ldb,
                      beta, golden[base + "/C"], ldc)
        assert np.array_equal(got, golden[key]), key
        checked += 1
    assert checked > 80
