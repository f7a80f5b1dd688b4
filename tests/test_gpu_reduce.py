"""Parity of global and per-axis reductions with the reference's Solid CPU library.

Bit-exact: every reduction with a bool, integer or counting result, and
minimum/maximum (and their _abs forms) on every type.  Floating-point sums,
products and norms accumulate in a different order than the OpenMP code, so they
are held to two bounds.  Against the reference: |got - want| <= tol * sqrt(n) *
scale with tol = 1e-5 (float, and half/chalf which accumulate in float), 1e-12
(double); scale is the sum of magnitudes (the natural condition of a sum) or the
value itself for norms.  That bound is wide (the reference's own sequential float
sum is that far from the exact value), so sum, sum_abs and norm2 are also held to
|got - f64| <= (4 log2 n + 4) u scale against a float64 evaluation of the same data
(util.accumulation_bound shows by arithmetic that a result missing 1 % of the
elements exceeds it at every size tested here).
"""
import numpy as np
import pytest

import util
from solid_b200 import dtypes as dt
from solid_b200 import oplist as ol

pytestmark = pytest.mark.gpu

FLOAT_ACCUM = {"sum", "sum_nan", "prod", "prod_nan", "sum_abs", "sum_abs_nan", "norm", "norm_nan", "norm2", "norm2_nan"}


def decode(raw: bytes, dtype: str):
    return np.frombuffer(raw[: dt.SIZE[dtype]], dtype=dt.NUMPY[dtype])


def close_enough(got, want, rdtype, n, scale, what, src_dtype=None):
    """Floating accumulations: tolerance scaled by sqrt(n); the half types also allow one
    unit in the last place of the stored result."""
    tol = 1e-12 if rdtype in ("double", "cdouble") else 1e-5
    g, w = util.as_float_components(got, rdtype), util.as_float_components(want, rdtype)
    both_nan = np.isnan(g) & np.isnan(w)
    same_inf = np.isinf(g) & np.isinf(w) & (np.sign(g) == np.sign(w))
    ok = both_nan | same_inf
    bound = tol * np.sqrt(max(n, 1)) * max(scale, 1e-30)
    if rdtype in ("half", "chalf"):
        bound = bound + np.abs(w) * 2.0 ** -10
    if src_dtype in dt.GROUPS["integer_bool"] and rdtype == "double":
        bound = bound + np.abs(w) * 1e-6          # integer norms go through the oracle's single-precision pow
    with np.errstate(invalid="ignore"):
        ok |= np.abs(g - w) <= bound
    assert ok.all(), "%s: got %r want %r (bound %g)" % (what, g, w, bound)


def input_kind(op):
    if op.startswith("prod"):
        return "near_one"
    return "special" if op.endswith("_nan") or op in ("any_nan", "any_inf", "all_finite") else "general"


def make_input(view, rng, op):
    kind = input_kind(op)
    if kind == "near_one":
        buf = util.fill_buffer(view, rng, "general")
        n = view.nbytes // dt.SIZE[view.dtype]
        if view.dtype in dt.GROUPS["float"]:
            comp = {"half": None, "chalf": None}.get(view.dtype, 0)
            vals = rng.uniform(0.97, 1.03, 2 * n + 2).astype(np.float32)
            if view.dtype in ("half", "chalf"):
                raw = util.f32_to_solid_half(vals).view(np.uint8)
            elif view.dtype in ("float", "cfloat"):
                raw = vals.view(np.uint8)
            else:
                raw = vals.astype(np.float64).view(np.uint8)
            if view.dtype in dt.COMPLEX:                # keep imaginary parts small
                c = np.frombuffer(raw.tobytes(), dtype={"chalf": np.uint16, "cfloat": np.float32, "cdouble": np.float64}[view.dtype]).copy()
                c[1::2] = 0
                raw = c.view(np.uint8)
            buf[:] = 0
            m = min(len(raw), len(buf)); buf[:m] = raw[:m]
        else:
            vals = rng.integers(1, 3, n + 1).astype(dt.NUMPY[view.dtype])
            if view.dtype == "bool":
                vals = (vals > 0).astype(np.uint8)
            raw = vals.view(np.uint8); buf[:] = 0; m = min(len(raw), len(buf)); buf[:m] = raw[:m]
        return buf
    return util.fill_buffer(view, rng, kind)


def reduce_views(dtype):
    es = dt.SIZE[dtype]
    out = [("n1", util.dense_view(dtype, [1])), ("n7", util.dense_view(dtype, [7])),
           ("n1000", util.dense_view(dtype, [1000])), ("n70001", util.dense_view(dtype, [70001])),
           ("offset", util.dense_view(dtype, [4097], offset_elems=1)),
           ("padded", util.dense_view(dtype, [100, 31], pad_elems=7)),
           ("scalar", util.dense_view(dtype, []))]
    v = util.dense_view(dtype, [9, 20, 11])
    out.append(("permuted", util.View(dtype, [11, 9, 20], [v.strides[2], v.strides[0], v.strides[1]], 0, v.nbytes)))
    out.append(("strided", util.View(dtype, [500], [3 * es], 0, 1500 * es + 64)))
    return out


ALL_GLOBAL = {**ol.REDUCE_BOOL_OPS, **ol.REDUCE_U64_OPS, **ol.REDUCE_VOID_OPS}


@pytest.mark.parametrize("op", sorted(ALL_GLOBAL))
def test_global_reduction_matches_reference(op, gpu, cpu):
    import torch
    dev = util.Device()
    scratch = dev.empty(gpu.reduce_all_buffer_size(1 << 24, 0) + 64)
    for dtype in dt.GROUPS[ALL_GLOBAL[op]]:
        if op == "nnz_nan" and dtype == "chalf":
            continue      # the reference converts the already converted float back through the half
                          # decoder (reduce_ops.h:283-284), so magnitudes below one count as zero there
        rdtype = ol.reduce_result_type(op, dtype)
        rng = np.random.default_rng(1000 + dt.INDEX[dtype])
        for name, v in reduce_views(dtype):
            buf = make_input(v, rng, op)
            want = decode(cpu.reduce_all(op, dtype, v.size, v.strides, buf.ctypes.data + v.offset), rdtype)
            d = dev.upload(buf)
            got = decode(gpu.reduce_all(op, dtype, v.size, v.strides, d.data_ptr() + v.offset, scratch.data_ptr(),
                                        dev.stream), rdtype)
            what = "%s_%s %s" % (op, dtype, name)
            if op in FLOAT_ACCUM and rdtype in dt.GROUPS["float"]:
                vals = util.as_float_components(util.gather(buf, v), dtype)
                vals = vals[np.isfinite(vals)]
                if op.startswith("prod"):
                    scale = float(np.abs(util.as_float_components(want, rdtype)).max()) * 4
                elif op.startswith("norm"):
                    scale = float(np.abs(util.as_float_components(want, rdtype)).max())
                else:
                    scale = float(np.abs(vals).sum())
                close_enough(got, want, rdtype, v.nelem, scale, what, dtype)
                if op in util.TIGHT_ACCUM and not (op.endswith("_nan") and dtype in dt.COMPLEX):
                    truth, tscale = util.f64_accumulate(op, util.as_values(util.gather(buf, v), dtype))
                    util.assert_accumulation(util.as_values(got, rdtype)[0], truth, v.nelem, rdtype, tscale, what)
            else:
                # complex magnitudes go through hypot, a library function: 2 ulp
                util.assert_same(got, want, rdtype, 2 if (dtype in dt.COMPLEX and op.endswith("_abs")) else 0, what)


@pytest.mark.parametrize("p", [1.0, 3.0, 0.5])
def test_global_norm_p(p, gpu, cpu):
    dev = util.Device()
    scratch = dev.empty(gpu.reduce_all_buffer_size(1 << 24, 0) + 64)
    for op in ("norm", "norm_nan"):
        for dtype in dt.NAMES:
            if dtype in dt.SINT:
                continue  # the reference stores p/2 and 1/p as integers into double fields for the signed
                          # types (solid/src/core/cpu/template_reduce_all.c:350-361) and returns 1
            rdtype = ol.reduce_result_type(op, dtype)
            rng = np.random.default_rng(5)
            v = util.dense_view(dtype, [5000])
            buf = util.fill_buffer(v, rng, "special" if op == "norm_nan" and dtype in dt.GROUPS["float"] else "general")
            want = decode(cpu.reduce_all(op, dtype, v.size, v.strides, buf.ctypes.data, p=p), rdtype)
            d = dev.upload(buf)
            got = decode(gpu.reduce_all(op, dtype, v.size, v.strides, d.data_ptr(), scratch.data_ptr(), dev.stream, p=p), rdtype)
            g, w = util.as_float_components(got, rdtype), util.as_float_components(want, rdtype)
            with np.errstate(invalid="ignore"):
                ok = (np.isnan(g) & np.isnan(w)) | (g == w) | (np.abs(g - w) <= 2e-3 * np.abs(w) + 1e-30)
            assert ok.all(), "%s_%s p=%g: got %r want %r" % (op, dtype, p, g, w)


def test_range_tests_match_reference(gpu, cpu):
    dev = util.Device()
    scratch = dev.empty(gpu.reduce_all_buffer_size(1 << 24, 0) + 64)
    rng = np.random.default_rng(9)
    for dtype in dt.NAMES:
        v = util.dense_view(dtype, [3001])
        buf = util.fill_buffer(v, rng, "general")
        vals = util.gather(buf, v)
        order = np.argsort(util.as_float_components(vals, dtype)[:: 2 if dtype in dt.COMPLEX else 1], kind="stable")
        lo, hi, mid = vals[order[0]].tobytes(), vals[order[-1]].tobytes(), vals[order[len(order) // 2]].tobytes()
        d = dev.upload(buf)
        for op in ol.REDUCE_BOUND1_OPS:
            for b in (lo, hi, mid):
                want = cpu.reduce_all(op, dtype, v.size, v.strides, buf.ctypes.data, bounds=(b,))[0]
                got = gpu.reduce_all(op, dtype, v.size, v.strides, d.data_ptr(), scratch.data_ptr(), dev.stream, bounds=(b,))[0]
                assert got == want, "%s_%s" % (op, dtype)
        for op in ol.REDUCE_BOUND2_OPS:
            for b1, b2 in ((lo, hi), (lo, mid), (mid, hi), (hi, lo)):
                want = cpu.reduce_all(op, dtype, v.size, v.strides, buf.ctypes.data, bounds=(b1, b2))[0]
                got = gpu.reduce_all(op, dtype, v.size, v.strides, d.data_ptr(), scratch.data_ptr(), dev.stream, bounds=(b1, b2))[0]
                assert got == want, "%s_%s" % (op, dtype)


def test_empty_tensor_results(gpu, cpu):
    """Empty tensors give the identity; minimum/maximum refuse them with an error."""
    from solid_b200._lib import SolidError
    dev = util.Device()
    scratch = dev.empty(1 << 16)
    d = dev.empty(64)
    host = np.zeros(64, dtype=np.uint8)
    for dtype in ("float", "int16", "bool", "cdouble"):
        for op in ("sum", "prod", "any", "all", "nnz", "norm2", "sum_abs"):
            rdtype = ol.reduce_result_type(op, dtype)
            want = decode(cpu.reduce_all(op, dtype, [0], [dt.SIZE[dtype]], host.ctypes.data), rdtype)
            got = decode(gpu.reduce_all(op, dtype, [0], [dt.SIZE[dtype]], d.data_ptr(), scratch.data_ptr(), dev.stream), rdtype)
            util.assert_same(got, want, rdtype, 0, "%s_%s empty" % (op, dtype))
        for op in ("maximum", "minimum", "maximum_abs", "minimum_abs"):
            with pytest.raises(SolidError):
                gpu.reduce_all(op, dtype, [3, 0], [dt.SIZE[dtype]] * 2, d.data_ptr(), scratch.data_ptr(), dev.stream)


# ---------------------------------------------------------------------------
AXIS_SHAPES = [((64, 50), (0,)), ((64, 50), (1,)), ((1000, 37), (0,)), ((37, 1000), (1,)), ((130, 700), (1,)),
               ((5, 6, 7), (1,)), ((5, 6, 7), (0, 2)), ((5, 6, 7), (0, 1, 2)), ((3, 2049), (1,)), ((4100, 3), (0,)),
               ((17,), (0,)), ((8, 9, 10, 3), (1, 2))]
ALL_AXIS = {**ol.AXIS_OPS}


@pytest.mark.parametrize("op", sorted(ALL_AXIS))
def test_axis_reduction_matches_reference(op, gpu, cpu):
    dev = util.Device()
    base = op[5:]
    for dtype in dt.GROUPS[ALL_AXIS[op]]:
        if base == "nnz_nan" and dtype == "chalf":
            continue      # see the global test
        rdtype = ol.reduce_result_type(op, dtype)
        rng = np.random.default_rng(2000 + dt.INDEX[dtype])
        for shape, axes in AXIS_SHAPES:
            if base.startswith("prod") and max(shape) > 200:
                continue
            for pad in (0, 3):
                v = util.dense_view(dtype, list(shape), pad_elems=pad)
                buf = make_input(v, rng, base)
                keep = [i for i in range(len(shape)) if i not in axes]
                size = [shape[i] for i in keep]; st1 = [v.strides[i] for i in keep]
                rsize = [shape[i] for i in axes]; rst = [v.strides[i] for i in axes]
                vo = util.dense_view(rdtype, size)
                out0 = np.zeros(vo.nbytes, dtype=np.uint8)
                want = out0.copy()
                cpu.reduce_axis(op, dtype, size, st1, buf.ctypes.data, vo.strides, want.ctypes.data, rsize, rst)
                d, do = dev.upload(buf), dev.upload(out0)
                cfg = gpu.reduce_axis_prepare(dt.WORKSIZE[rdtype], size, st1, d.data_ptr(), vo.strides, do.data_ptr(),
                                              rsize, rst, dev.stream)
                scratch = dev.empty(cfg.bufferSize + 16)
                cfg.data.ptrBuffer = scratch.data_ptr() if cfg.bufferSize else None
                gpu.reduce_axis(op, dtype, cfg)
                got = dev.download(do)
                what = "%s_%s shape %s axes %s pad %d" % (op, dtype, shape, axes, pad)
                g, w = util.gather(got, vo), util.gather(want, vo)
                if base in FLOAT_ACCUM and rdtype in dt.GROUPS["float"]:
                    n = int(np.prod(rsize))
                    mags = np.abs(util.as_float_components(util.gather(buf, v), dtype))
                    mags = mags[np.isfinite(mags)]
                    if base.startswith("prod") or base.startswith("norm"):
                        scale = float(np.abs(util.as_float_components(w, rdtype)).max()) * 4
                    else:
                        scale = float(mags.max() * n) if mags.size else 1.0
                    close_enough(g, w, rdtype, n, scale, what, dtype)
                    if base in util.TIGHT_ACCUM and not (base.endswith("_nan") and dtype in dt.COMPLEX):
                        arr = util.as_values(util.gather(buf, v), dtype).reshape(shape, order="F")
                        truth, tscale = util.f64_accumulate(base, arr, axis=tuple(axes))
                        util.assert_accumulation(util.as_values(g, rdtype).reshape(truth.shape, order="F"), truth, n,
                                                 rdtype, tscale, what)
                else:
                    util.assert_same(g, w, rdtype, 2 if (dtype in dt.COMPLEX and base.endswith("_abs")) else 0, what)


def test_axis_norm_p(gpu, cpu):
    dev = util.Device()
    rng = np.random.default_rng(3)
    for dtype in ("float", "double", "uint16", "cfloat", "half"):
        rdtype = ol.reduce_result_type("axis_norm", dtype)
        v = util.dense_view(dtype, [300, 40])
        buf = util.fill_buffer(v, rng)
        for axes in ((0,), (1,)):
            keep = [i for i in range(2) if i not in axes]
            size = [v.size[i] for i in keep]; st1 = [v.strides[i] for i in keep]
            rsize = [v.size[i] for i in axes]; rst = [v.strides[i] for i in axes]
            vo = util.dense_view(rdtype, size)
            want = np.zeros(vo.nbytes, dtype=np.uint8)
            cpu.reduce_axis("axis_norm", dtype, size, st1, buf.ctypes.data, vo.strides, want.ctypes.data, rsize, rst, p=3.0)
            d, do = dev.upload(buf), dev.upload(np.zeros(vo.nbytes, dtype=np.uint8))
            cfg = gpu.reduce_axis_prepare(dt.WORKSIZE[rdtype], size, st1, d.data_ptr(), vo.strides, do.data_ptr(), rsize, rst, dev.stream)
            scratch = dev.empty(cfg.bufferSize + 16)
            cfg.data.ptrBuffer = scratch.data_ptr() if cfg.bufferSize else None
            gpu.reduce_axis("axis_norm", dtype, cfg, p=3.0)
            g = util.as_float_components(util.gather(dev.download(do), vo), rdtype)
            w = util.as_float_components(util.gather(want, vo), rdtype)
            with np.errstate(invalid="ignore"):
                ok = (np.isnan(g) & np.isnan(w)) | (g == w) | (np.abs(g - w) <= 2e-3 * np.abs(w) + 1e-30)
            assert ok.all(), "axis_norm_%s axes %s" % (dtype, axes)


@pytest.mark.gpu
def test_global_reductions_on_several_streams(gpu, cpu):
    """Split global reductions fold their partials in the last block to arrive, which is found through a
    counter kept per stream: interleave host-returning and device-resident calls on four streams
    (the default one included) and repeat them, so that every counter is used again after it was reset."""
    import torch
    dev = util.Device()
    rng = np.random.default_rng(77)
    n = (1 << 20) + 17
    hosts = [rng.integers(-1000, 1000, n).astype(np.int32) for _ in range(4)]
    want = [decode(cpu.reduce_all("sum", "int32", [n], [4], h.ctypes.data), "int64") for h in hosts]
    wmax = [decode(cpu.reduce_all("maximum", "int32", [n], [4], h.ctypes.data), "int32") for h in hosts]
    data = [dev.upload(h.view(np.uint8)) for h in hosts]
    streams = [torch.cuda.current_stream()] + [torch.cuda.Stream() for _ in range(3)]
    scratch = [dev.empty(gpu.reduce_all_buffer_size(n, 0) + 64) for _ in range(4)]
    results = [dev.empty(16) for _ in range(4)]
    torch.cuda.synchronize()
    for _ in range(5):
        for k in range(4):      # device-resident: nothing waits, the four streams overlap
            gpu.reduce_all_device("sum", "int32", [n], [4], data[k].data_ptr(), results[k].data_ptr(),
                                  scratch[k].data_ptr(), streams[k].cuda_stream)
        for k in range(4):      # host-returning on the same streams, queued behind the calls above
            got = decode(gpu.reduce_all("maximum", "int32", [n], [4], data[k].data_ptr(), scratch[k].data_ptr(),
                                        streams[k].cuda_stream), "int32")
            assert got == wmax[k], ("maximum", k)
        torch.cuda.synchronize()
        for k in range(4):
            got = dev.download(results[k])[:8].view(np.int64)[0]
            assert got == want[k][0], ("sum", k)
