"""Parity of the fused entry points with the kernel SEQUENCES the reference runs for the same
expressions (each operand converted into a temporary of the common type with Tensor_copy, then
Tensor_scale, Tensor_add, and a final converting copy), on the reference's Solid CPU library.
Elementwise results are bit-exact; the two sums of axpy_sums are held to (4 log2 n + 4) u sum|z| against a
float64 evaluation, and to the tolerance of the floating-point reductions (1e-5 * sqrt(n) * sum|z| for float,
1e-12 for double) against the reference's own sum and norm2 of z."""
import numpy as np
import pytest

import util
from solid_b200 import dtypes as dt

pytestmark = pytest.mark.gpu


def cpu_convert(cpu, src, dst, view, buf, swapped, n_total):
    """Dense array of `dst` values of a (possibly byteswapped / strided / unaligned) view, by the reference copy."""
    out = np.zeros(n_total, dtype=dt.NUMPY[dst])
    dense = util.dense_view(dst, view.size)
    cpu.copy(src, dst, view.size, view.strides, buf.ctypes.data + view.offset, view.size, dense.strides, out.ctypes.data,
             variant="byteswap_copy" if swapped else "copy")
    return out


MIXED_CASES = [
    # (ctype, dst, (ta, swapped), (tb, swapped), (tc, swapped))
    ("double", "float", ("double", False), ("int32", True), ("float", False)),
    ("double", "double", ("float", True), ("int16", False), ("double", True)),
    ("float", "half", ("half", False), ("uint8", False), ("float", False)),
    ("double", "int32", ("int64", False), ("double", False), ("int8", False)),
    ("float", "float", ("float", False), ("float", False), ("float", False)),
    ("double", "cfloat", ("cdouble", False), ("uint16", True), ("half", True)),
]


@pytest.mark.parametrize("case", MIXED_CASES)
def test_mixed_multiply_add_matches_reference_sequence(case, gpu, cpu):
    ctype, dst, (ta, sa), (tb, sb), (tc, sc) = case
    dev = util.Device()
    rng = np.random.default_rng(5)
    # (130, 70) and (96, 192) hold interior tiles (the unrolled path) as well as edge tiles; "swapped_dst" stores the
    # result with reversed bytes; the 3-d case keeps a third dimension that cannot be merged (padded planes)
    for shape, layout in (((130, 70), "transposed_a"), ((64, 64), "dense"), ((33, 17, 3), "dense"),
                          ((4099,), "dense"), ((96, 40), "broadcast_c"), ((70, 50), "unaligned_b"),
                          ((96, 192), "transposed_a swapped_dst"), ((70, 130, 3), "transposed_a planes"),
                          ((64, 128), "dense_2d_padded swapped_dst")):
        n = int(np.prod(shape))
        sd = "swapped_dst" in layout
        # views
        if "transposed_a" in layout:
            es_a = dt.SIZE[ta]
            if len(shape) == 2:
                va = util.View(ta, list(shape), [shape[1] * es_a, es_a], 0, n * es_a)
            else:                                    # planes of transposed matrices, 5 elements of padding between planes
                plane = (shape[0] * shape[1] + 5) * es_a
                va = util.View(ta, list(shape), [shape[1] * es_a, es_a, plane], 0, plane * shape[2])
        else:
            va = util.dense_view(ta, list(shape))
        vb = util.dense_view(tb, list(shape), pad_elems=3 if len(shape) > 1 else 0)
        if layout == "unaligned_b":
            eb = dt.SIZE[tb]
            vb = util.View(tb, list(shape), [eb, shape[0] * eb + 1], 1, (shape[0] * eb + 1) * shape[1] + 64)
        if layout == "broadcast_c":
            vc = util.View(tc, list(shape), [0, dt.SIZE[tc]], 0, shape[1] * dt.SIZE[tc] + 64)
        else:
            vc = util.dense_view(tc, list(shape))
        vd = util.dense_view(dst, list(shape), pad_elems=2 if "padded" in layout else 0)
        kind = "small" if (dst in dt.GROUPS["integer"] or ta in dt.SINT) else "general"
        bufs = []
        for v, sw in ((va, sa), (vb, sb), (vc, sc)):
            b = util.fill_buffer(v, rng, kind)
            if sw:                                    # store the logical values with reversed bytes
                from test_gpu_copy import swap_buffer
                b = swap_buffer(b, v.dtype, v)
            bufs.append(b)
        # reference sequence
        A = cpu_convert(cpu, ta, ctype, va, bufs[0], sa, n)
        B = cpu_convert(cpu, tb, ctype, vb, bufs[1], sb, n)
        Cc = cpu_convert(cpu, tc, ctype, vc, bufs[2], sc, n)
        es = dt.SIZE[ctype]
        P, S = np.zeros(n, dtype=dt.NUMPY[ctype]), np.zeros(n, dtype=dt.NUMPY[ctype])
        cpu.binary("multiply", ctype, [n], [es], A.ctypes.data, [es], B.ctypes.data, [es], P.ctypes.data)
        cpu.binary("add", ctype, [n], [es], P.ctypes.data, [es], Cc.ctypes.data, [es], S.ctypes.data)
        want = np.zeros(n * dt.SIZE[dst], dtype=np.uint8)
        cpu.copy(ctype, dst, [n], [es], S.ctypes.data, [n], [dt.SIZE[dst]], want.ctypes.data)
        if sd:
            from test_gpu_copy import swap_buffer
            want = swap_buffer(want, dst, util.dense_view(dst, [n]))
        # fused kernel
        d = [dev.upload(b) for b in bufs]
        dd = dev.upload(np.zeros(vd.nbytes, dtype=np.uint8))
        gpu.mixed_multiply_add(list(shape), [(d[0].data_ptr() + va.offset, va.strides, ta, sa),
                                             (d[1].data_ptr() + vb.offset, vb.strides, tb, sb),
                                             (d[2].data_ptr() + vc.offset, vc.strides, tc, sc),
                                             (dd.data_ptr(), vd.strides, dst, sd)], ctype, dev.stream)
        got = dev.download(dd)
        elems = util.gather(got, vd)                 # column-major elements of the (possibly padded) destination
        untouched = got.copy()
        esd = dt.SIZE[dst]
        idx = np.zeros(1, dtype=np.int64)
        for sz, st in zip(vd.size, vd.strides):
            idx = (np.arange(sz, dtype=np.int64)[:, None] * st + idx[None, :]).reshape(-1)
        untouched[(idx[:, None] + np.arange(esd)[None, :]).reshape(-1)] = 0
        assert not untouched.any(), "bytes outside the destination's elements were written (%s %s)" % (case, layout)
        got = elems.view(np.uint8)
        if sd:                                       # compare the stored bytes: NaN payloads do not arise in these cases
            assert np.array_equal(got, want), "%s %s %s" % (case, shape, layout)
            continue
        # same bits, except that two NaNs count as equal whatever their payload (rows of the unaligned
        # operand reinterpret neighbouring bytes, which may happen to be NaN patterns)
        g = got[: n * dt.SIZE[dst]].view(dt.NUMPY[dst]); w = want[: n * dt.SIZE[dst]].view(dt.NUMPY[dst])
        util.assert_same(g, w, dst, 0, "%s %s %s" % (case, shape, layout))


@pytest.mark.parametrize("dtype", ["half", "float", "double"])
def test_axpy_matches_scale_then_add(dtype, gpu, cpu):
    dev = util.Device()
    rng = np.random.default_rng(8)
    es = dt.SIZE[dtype]
    for size, pad in (([4099], 0), ([100, 37], 5), ([], 0), ([0], 0)):
        v = util.dense_view(dtype, size, pad_elems=pad)
        x, y = util.fill_buffer(v, rng), util.fill_buffer(v, rng)
        a = util.random_values(dtype, 1, rng)
        t, want = np.zeros_like(x), util.fill_buffer(v, rng)
        z0 = want.copy()
        cpu.binary("multiply", dtype, size, v.strides, x.ctypes.data, [0] * len(size), a.ctypes.data, v.strides, t.ctypes.data)
        cpu.binary("add", dtype, size, v.strides, t.ctypes.data, v.strides, y.ctypes.data, v.strides, want.ctypes.data)
        dx, dy, dz = dev.upload(x), dev.upload(y), dev.upload(z0)
        gpu.axpy(dtype, size, a.tobytes(), v.strides, dx.data_ptr(), v.strides, dy.data_ptr(), v.strides, dz.data_ptr(), dev.stream)
        assert np.array_equal(dev.download(dz), want), (dtype, size)


@pytest.mark.parametrize("dtype", ["float", "double"])
def test_axpy_sums_matches_reference_sequence(dtype, gpu, cpu):
    import torch
    dev = util.Device()
    rng = np.random.default_rng(9)
    es = dt.SIZE[dtype]
    for n in (1, 5, 4096, 1000003, (1 << 24) + 3):      # the last one needs the two-level fold of the partials
        part = dev.empty(gpu.axpy_sums_buffer_size(0, n))
        x = rng.uniform(-1, 1, n).astype(dt.NUMPY[dtype]); y = rng.uniform(-1, 1, n).astype(dt.NUMPY[dtype])
        a = np.array([0.5], dtype=dt.NUMPY[dtype])
        t, z = np.zeros_like(x), np.zeros_like(x)
        cpu.binary("multiply", dtype, [n], [es], x.ctypes.data, [0], a.ctypes.data, [es], t.ctypes.data)
        cpu.binary("add", dtype, [n], [es], t.ctypes.data, [es], y.ctypes.data, [es], z.ctypes.data)
        dx, dy = dev.upload(x.view(np.uint8)), dev.upload(y.view(np.uint8))
        dz = dev.empty(n * es); sums = dev.empty(2 * es)
        gpu.axpy_sums(dtype, n, a.tobytes(), dx.data_ptr(), dy.data_ptr(), dz.data_ptr(), sums.data_ptr(), part.data_ptr(), dev.stream)
        got_z = dev.download(dz)[: n * es].view(dt.NUMPY[dtype])
        assert np.array_equal(got_z, z), (dtype, n)
        got = dev.download(sums)[: 2 * es].view(dt.NUMPY[dtype]).astype(np.float64)
        z64 = z.astype(np.float64)
        tol = (1e-5 if dtype == "float" else 1e-12) * np.sqrt(n)
        # against a float64 evaluation: the bound of a tree of short chains (util.accumulation_bound)
        assert abs(got[0] - z64.sum()) <= util.accumulation_bound(n, dtype, np.abs(z64).sum()) + 1e-300
        assert abs(got[1] - (z64 ** 2).sum()) <= util.accumulation_bound(n, dtype, (z64 ** 2).sum()) + 1e-300
        # and against the reference's own sum / norm2 of z
        s_ref = np.frombuffer(cpu.reduce_all("sum", dtype, [n], [es], z.ctypes.data)[:es], dtype=dt.NUMPY[dtype])[0]
        q_ref = np.frombuffer(cpu.reduce_all("norm2", dtype, [n], [es], z.ctypes.data)[:es], dtype=dt.NUMPY[dtype])[0]
        assert abs(got[0] - float(s_ref)) <= 2 * tol * np.abs(z64).sum() + 1e-300
        assert abs(np.sqrt(got[1]) - float(q_ref)) <= 2 * tol * float(q_ref) + 1e-300


def test_device_resident_reduction_matches_host_returning_form(gpu):
    dev = util.Device()
    rng = np.random.default_rng(10)
    scratch = dev.empty(gpu.reduce_all_buffer_size(1 << 22, 0) + 64)
    for dtype, op in (("float", "sum"), ("double", "norm2"), ("int32", "maximum"), ("bool", "nnz"), ("uint8", "any")):
        v = util.dense_view(dtype, [100003])
        buf = util.fill_buffer(v, rng)
        d = dev.upload(buf)
        host = gpu.reduce_all(op, dtype, v.size, v.strides, d.data_ptr(), scratch.data_ptr(), dev.stream)
        res = dev.empty(16)
        gpu.reduce_all_device(op, dtype, v.size, v.strides, d.data_ptr(), res.data_ptr(), scratch.data_ptr(), dev.stream)
        from solid_b200 import oplist as ol
        k = dt.SIZE[ol.reduce_result_type(op, dtype)]
        assert bytes(dev.download(res)[:k]) == host[:k], (dtype, op)


def test_axpy_half_every_pattern(gpu, cpu):
    """Half axpy takes a vector-wide shortcut while all products and sums stay in the normal half range and
    falls back per vector otherwise: run every half bit pattern as x against scalars and addends that keep
    most vectors on the shortcut (ordinary magnitudes), push them to its edges (tiny and huge scalars,
    cancelling addends) or leave it (zeros, infinities, NaNs)."""
    dev = util.Device()
    rng = np.random.default_rng(81)
    n = 1 << 16
    x = np.arange(n, dtype=np.uint16)
    addends = {
        "ordinary": (rng.integers(0x3000, 0x4800, n) | (rng.integers(0, 2, n) << 15)).astype(np.uint16),   # 0.125 .. 8, both signs
        "cancelling": (x ^ 0x8000).astype(np.uint16),                                                        # y = -x
        "any": rng.permutation(n).astype(np.uint16),
        "zero": np.zeros(n, dtype=np.uint16),
    }
    for a_bits in (0x3800, 0x3C01, 0xC200, 0x1400, 0x63D0, 0x0000, 0x7C00):    # 0.5, 1+ulp, -3, 2^-10, 1000, 0, inf
        a = np.array([a_bits], dtype=np.uint16)
        for name, y in addends.items():
            t, want = np.zeros(n, dtype=np.uint16), np.zeros(n, dtype=np.uint16)
            cpu.binary("multiply", "half", [n], [2], x.ctypes.data, [0], a.ctypes.data, [2], t.ctypes.data)
            cpu.binary("add", "half", [n], [2], t.ctypes.data, [2], y.ctypes.data, [2], want.ctypes.data)
            dx, dy, dz = dev.upload(x.view(np.uint8)), dev.upload(y.view(np.uint8)), dev.empty(2 * n)
            gpu.axpy("half", [n], a.tobytes(), [2], dx.data_ptr(), [2], dy.data_ptr(), [2], dz.data_ptr(), dev.stream)
            got = dev.download(dz)[: 2 * n].view(np.uint16)
            bad = np.nonzero(got != want)[0]
            assert bad.size == 0, (hex(a_bits), name, [(hex(x[i]), hex(y[i]), hex(got[i]), hex(want[i])) for i in bad[:5]])
