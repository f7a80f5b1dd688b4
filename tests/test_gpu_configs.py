"""Parity at the benchmark configurations' own sizes.

The layout sweeps of the other test files use small tensors; the shapes whose throughput bench.py reports take
other paths through the launch logic (grid sizes in the hundreds of thousands, split axis reductions with a second
pass, the single-launch global reduction over a full wave of blocks, 64-bit element counts).  Each configuration is
therefore run once at its named size on seeded data (numpy Generator(PCG64(seed)); the 2^32-element case uses the
counter hash of bench.py, which needs no host copy) and compared, through the C-ABI, with the reference's Solid CPU
library on the same buffers:

  bit-exact   integer / bool results, minimum / maximum, copy / convert / byte order, IEEE add / multiply (also
              complex multiply, conj), sqrt, fabs, the fused kernels' elementwise output against the reference's
              SEQUENCE of kernels
  <= 2 ulp    exp, log, sin (float), hypot inside absolute (cdouble)
  sums, norms |got - reference| <= tol sqrt(n) scale, tol = 1e-5 (float) / 1e-12 (double), AND
              |got - float64 evaluation| <= (4 log2 n + 4) u scale  (util.accumulation_bound)
"""
import json
import os
from pathlib import Path

import numpy as np
import pytest

import util
from solid_b200 import dtypes as dt

pytestmark = pytest.mark.gpu

GOLDEN = Path(__file__).resolve().parent / "golden"


@pytest.fixture()
def cpu_all(cpu):
    """The oracle on every host core for elementwise work and single-axis reductions (their results do not depend
    on the thread count, except float sums, which are compared with a tolerance anyway); the session default of
    one thread is restored afterwards."""
    cpu.set_threads(os.cpu_count() or 1)
    yield cpu
    cpu.set_threads(1)


def gen(seed):
    return np.random.Generator(np.random.PCG64(seed))


def raw(a):
    return np.ascontiguousarray(a).view(np.uint8).reshape(-1)


def scalar(raw16: bytes, dtype: str):
    return np.frombuffer(raw16[: dt.SIZE[dtype]], dtype=dt.NUMPY[dtype])[0]


def check_float_reduction(op, got, want, x64, n, rdtype, what):
    """Both bounds of the module docstring for one floating-point sum or norm."""
    tol = 1e-12 if rdtype == "double" else 1e-5
    truth, scale = util.f64_accumulate(op, x64)
    assert abs(float(got) - float(want)) <= tol * np.sqrt(n) * float(scale), "%s against the reference: %r %r" % (what, got, want)
    util.assert_accumulation(np.float64(got), truth, n, rdtype, scale, what + " against float64")


# ---------------------------------------------------------------------------------------------------------------
def test_c1_float_2p24(gpu, cpu_all):
    cpu = cpu_all
    dev = util.Device()
    n = 1 << 24
    x = gen(0xC1A0).uniform(-1, 1, n).astype(np.float32)
    y = gen(0xC1A1).uniform(-1, 1, n).astype(np.float32)
    dx, dy, dz = dev.upload(raw(x)), dev.upload(raw(y)), dev.empty(4 * n)
    want = np.empty(n, dtype=np.float32)
    for op in ("add", "multiply"):
        cpu.binary(op, "float", [n], [4], x.ctypes.data, [4], y.ctypes.data, [4], want.ctypes.data)
        gpu.binary(op, "float", [n], [4], dx.data_ptr(), [4], dy.data_ptr(), [4], dz.data_ptr(), dev.stream)
        got = dev.download(dz)[: 4 * n].view(np.float32)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), op
    scratch = dev.empty(gpu.reduce_all_buffer_size(n, 0) + 64)
    x64 = x.astype(np.float64)
    for op in ("sum", "norm2"):
        w = scalar(cpu.reduce_all(op, "float", [n], [4], x.ctypes.data), "float")
        g = scalar(gpu.reduce_all(op, "float", [n], [4], dx.data_ptr(), scratch.data_ptr(), dev.stream), "float")
        check_float_reduction(op, g, w, x64, n, "float", "C1 " + op)
        # the device-resident form runs the same kernel: same bits
        res = dev.empty(16)
        gpu.reduce_all_device(op, "float", [n], [4], dx.data_ptr(), res.data_ptr(), scratch.data_ptr(), dev.stream)
        assert dev.download(res)[:4].view(np.float32)[0].tobytes() == np.float32(g).tobytes(), op
    w = cpu.reduce_all("maximum", "float", [n], [4], x.ctypes.data)[:4]
    g = gpu.reduce_all("maximum", "float", [n], [4], dx.data_ptr(), scratch.data_ptr(), dev.stream)[:4]
    assert g == w and scalar(g, "float") == x.max(), "maximum"


# ---------------------------------------------------------------------------------------------------------------
def test_c2_mixed_layout_binary_4096(gpu, cpu_all):
    """C(float) = A(double, transposed view) * B(int32, stored byte-reversed) + r(float, 1 x 4096 broadcast), against
    the reference's sequence: three converting copies into dense doubles, multiply, add, double -> float copy."""
    cpu = cpu_all
    dev = util.Device()
    m = 4096
    n = m * m
    A = gen(0xC2A0).uniform(-1, 1, (m, m))                          # row-major buffer; the tensor is its transpose
    B = gen(0xC2A1).integers(-1000, 1001, (m, m)).astype(np.int32)  # column-major element order below
    r = gen(0xC2A2).uniform(-1, 1, m).astype(np.float32)
    Bsw = B.astype(">i4")
    sA, sB, sr, sD = [8 * m, 8], [4, 4 * m], [0, 4], [8, 8 * m]
    a64, b64, r64 = (np.empty(n, dtype=np.float64) for _ in range(3))
    cpu.copy("double", "double", [m, m], sA, A.ctypes.data, [m, m], sD, a64.ctypes.data)
    cpu.copy("int32", "double", [m, m], sB, Bsw.ctypes.data, [m, m], sD, b64.ctypes.data, variant="byteswap_copy")
    cpu.copy("float", "double", [m, m], sr, r.ctypes.data, [m, m], sD, r64.ctypes.data)
    p, s = np.empty(n, dtype=np.float64), np.empty(n, dtype=np.float64)
    cpu.binary("multiply", "double", [n], [8], a64.ctypes.data, [8], b64.ctypes.data, [8], p.ctypes.data)
    cpu.binary("add", "double", [n], [8], p.ctypes.data, [8], r64.ctypes.data, [8], s.ctypes.data)
    want = np.empty(n, dtype=np.float32)
    cpu.copy("double", "float", [n], [8], s.ctypes.data, [n], [4], want.ctypes.data)
    # a sanity anchor independent of the reference: the same expression in numpy
    assert np.array_equal(want, (A.reshape(-1, order="F") * B.reshape(-1).astype(np.float64)
                                 + np.repeat(r.astype(np.float64), m)).astype(np.float32))
    dA, dB, dr, dC = dev.upload(raw(A)), dev.upload(raw(Bsw)), dev.upload(raw(r)), dev.empty(4 * n)
    gpu.mixed_multiply_add([m, m], [(dA.data_ptr(), sA, "double", False), (dB.data_ptr(), sB, "int32", True),
                                    (dr.data_ptr(), sr, "float", False), (dC.data_ptr(), [4, 4 * m], "float", False)],
                           "double", dev.stream)
    got = dev.download(dC)[: 4 * n].view(np.float32)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), "fused mixed multiply-add"

    # the unfused operations on the same layouts, each against its reference counterpart
    d64 = dev.empty(8 * n)
    gpu.copy("double", "double", [m, m], sA, dA.data_ptr(), [m, m], sD, d64.data_ptr(), dev.stream)
    assert np.array_equal(dev.download(d64)[: 8 * n].view(np.float64), a64), "transposing copy"
    gpu.copy("int32", "double", [m, m], sB, dB.data_ptr(), [m, m], sD, d64.data_ptr(), dev.stream, variant="byteswap_copy")
    assert np.array_equal(dev.download(d64)[: 8 * n].view(np.float64), b64), "byte-reversed int32 -> double"
    # A^T + A with both operands double: one operand dense along the other dimension
    At = np.ascontiguousarray(A)                                    # second operand: column-major dense
    cpu.binary("add", "double", [m, m], sA, A.ctypes.data, sD, At.ctypes.data, sD, s.ctypes.data)
    dAt = dev.upload(raw(At))
    gpu.binary("add", "double", [m, m], sA, dA.data_ptr(), sD, dAt.data_ptr(), sD, d64.data_ptr(), dev.stream)
    assert np.array_equal(dev.download(d64)[: 8 * n].view(np.float64), s), "transposed operand add"


def test_c2_unaligned_byteswapped_double_to_half_4096(gpu, cpu_all):
    cpu = cpu_all
    dev = util.Device()
    n = 4096 * 4096
    v = gen(0xC2B0).uniform(-4, 4, n)
    buf = np.zeros(8 * n + 64, dtype=np.uint8)
    buf[3: 3 + 8 * n] = raw(v.astype(">f8"))
    want = np.empty(n, dtype=np.uint16)
    cpu.copy("double", "half", [n], [8], buf.ctypes.data + 3, [n], [2], want.ctypes.data, variant="byteswap_copy")
    d, dh = dev.upload(buf), dev.empty(2 * n)
    gpu.copy("double", "half", [n], [8], d.data_ptr() + 3, [n], [2], dh.data_ptr(), dev.stream, variant="byteswap_copy")
    got = dev.download(dh)[: 2 * n].view(np.uint16)
    assert np.array_equal(got, want)
    # as a 4096 x 4096 matrix (two dimensions, merged by the library) through copy_ex as well
    SOLID_GPU_COPY_SRC_SWAPPED = 1                                  # include/solid_core_gpu.h
    dh2 = dev.empty(2 * n)
    gpu.copy_ex("double", "half", SOLID_GPU_COPY_SRC_SWAPPED, [4096, 4096], [8, 8 * 4096], d.data_ptr() + 3,
                [4096, 4096], [2, 2 * 4096], dh2.data_ptr(), dev.stream)
    assert np.array_equal(dev.download(dh2)[: 2 * n].view(np.uint16), want)


# ---------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float", "int64"])
def test_c3_axis_reductions_8192(dtype, gpu, cpu_all):
    cpu = cpu_all
    dev = util.Device()
    k = 8192
    if dtype == "float":
        h = gen(0xC3A0).standard_normal((k, k), dtype=np.float32)
    else:
        h = gen(0xC3A1).integers(-2 ** 20, 2 ** 20, (k, k), dtype=np.int64, endpoint=True)
    es = dt.SIZE[dtype]
    # h is a C-order numpy array; as a column-major Ocean tensor its axis 0 (dense) is numpy's last axis
    strides = [es, es * k]
    d = dev.upload(raw(h))
    col_major = h.T                                                   # element [i, j] of the Ocean tensor
    x64 = col_major.astype(np.float64) if dtype == "float" else None
    for op in ("sum", "minimum", "maximum", "norm2"):
        rdtype = dtype if op != "norm2" else ("float" if dtype == "float" else "double")
        for axis in (0, 1):
            keep = 1 - axis
            vo = [dt.SIZE[rdtype]]
            want = np.zeros(k, dtype=dt.NUMPY[rdtype])
            cpu.reduce_axis("axis_" + op, dtype, [k], [strides[keep]], h.ctypes.data, vo, want.ctypes.data, [k], [strides[axis]])
            do = dev.empty(k * dt.SIZE[rdtype])
            cfg = gpu.reduce_axis_prepare(dt.WORKSIZE[rdtype], [k], [strides[keep]], d.data_ptr(), vo, do.data_ptr(),
                                          [k], [strides[axis]], dev.stream)
            scratch = dev.empty(cfg.bufferSize + 16)
            cfg.data.ptrBuffer = scratch.data_ptr() if cfg.bufferSize else None
            gpu.reduce_axis("axis_" + op, dtype, cfg)
            got = dev.download(do)[: k * dt.SIZE[rdtype]].view(dt.NUMPY[rdtype])
            what = "C3 axis_%s %s axis %d" % (op, dtype, axis)
            if dtype == "int64" and op != "norm2":
                assert np.array_equal(got, want), what
                ref = {"sum": col_major.sum(axis=axis), "minimum": col_major.min(axis=axis), "maximum": col_major.max(axis=axis)}[op]
                assert np.array_equal(got, ref), what + " (numpy)"
            elif op in ("minimum", "maximum"):
                assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), what
            elif dtype == "int64":                                       # norm2 of integers: double accumulation
                truth = np.sqrt((col_major.astype(np.float64) ** 2).sum(axis=axis))
                assert np.all(np.abs(got - want) <= 1e-12 * np.sqrt(k) * truth), what
                util.assert_accumulation(got, truth, k, "double", truth, what)
            else:
                truth, scale = util.f64_accumulate(op, x64, axis=axis)
                assert np.all(np.abs(got.astype(np.float64) - want.astype(np.float64)) <= 1e-5 * np.sqrt(k) * scale), what
                util.assert_accumulation(got, truth, k, "float", scale, what)


def test_c3_bool_mask_8192(gpu, cpu_all):
    cpu = cpu_all
    dev = util.Device()
    k = 8192
    n = k * k
    mask = (gen(0xC3B0).random(n) < 0.1).astype(np.uint8)
    d = dev.upload(mask)
    scratch = dev.empty(gpu.reduce_all_buffer_size(n, 0) + 64)
    for data, dd, label in ((mask, d, "p=0.1"),):
        for op, rdtype in (("any", "bool"), ("all", "bool"), ("nnz", "uint64")):
            for size, strides in (([n], [1]), ([k, k], [1, k])):
                w = cpu.reduce_all(op, "bool", size, strides, data.ctypes.data)[: dt.SIZE[rdtype]]
                g = gpu.reduce_all(op, "bool", size, strides, dd.data_ptr(), scratch.data_ptr(), dev.stream)[: dt.SIZE[rdtype]]
                assert g == w, (op, label, size)
    assert scalar(gpu.reduce_all("nnz", "bool", [n], [1], d.data_ptr(), scratch.data_ptr(), dev.stream), "uint64") == int(mask.sum())
    # the other answers of any / all: an all-false and an all-true mask, and a single differing element at the end
    zeros, ones = dev.upload(np.zeros(n, dtype=np.uint8)), dev.upload(np.ones(n, dtype=np.uint8))
    assert gpu.reduce_all("any", "bool", [n], [1], zeros.data_ptr(), scratch.data_ptr(), dev.stream)[0] == 0
    assert gpu.reduce_all("all", "bool", [n], [1], ones.data_ptr(), scratch.data_ptr(), dev.stream)[0] == 1
    zeros[n - 1] = 1
    ones[n - 1] = 0
    assert gpu.reduce_all("any", "bool", [n], [1], zeros.data_ptr(), scratch.data_ptr(), dev.stream)[0] == 1
    assert gpu.reduce_all("all", "bool", [n], [1], ones.data_ptr(), scratch.data_ptr(), dev.stream)[0] == 0


# ---------------------------------------------------------------------------------------------------------------
def test_c4_float_unary_2p26(gpu, cpu_all):
    cpu = cpu_all
    dev = util.Device()
    n = 1 << 26
    x = gen(0xC4A0).uniform(0.01, 10, n).astype(np.float32)
    dx, dy = dev.upload(raw(x)), dev.empty(4 * n)
    want = np.empty(n, dtype=np.float32)
    for op, ulp in (("sqrt", 0), ("exp", 2), ("log", 2), ("sin", 2), ("fabs", 0)):
        cpu.unary(op, "float", [n], [4], x.ctypes.data, [4], want.ctypes.data)
        gpu.unary(op, "float", [n], [4], dx.data_ptr(), [4], dy.data_ptr(), dev.stream)
        got = dev.download(dy)[: 4 * n].view(np.float32)
        if ulp == 0:
            assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), op
        else:
            dist = util.ulp_distance(got, want, "float")
            assert int(dist.max()) <= ulp, "%s: %d ulp at x = %r" % (op, int(dist.max()), x[int(dist.argmax())])


def test_c4_cdouble_2p26(gpu, cpu_all):
    cpu = cpu_all
    dev = util.Device()
    n = 1 << 26
    g1, g2 = gen(0xC4B0), gen(0xC4B1)
    a = np.empty(n, dtype=np.complex128)
    b = np.empty(n, dtype=np.complex128)
    a.real, a.imag = g1.standard_normal(n), g1.standard_normal(n)
    b.real, b.imag = g2.standard_normal(n), g2.standard_normal(n)
    da, db, dz = dev.upload(raw(a)), dev.upload(raw(b)), dev.empty(16 * n)
    want = np.empty(n, dtype=np.complex128)
    cpu.unary("conj", "cdouble", [n], [16], a.ctypes.data, [16], want.ctypes.data)
    gpu.unary("conj", "cdouble", [n], [16], da.data_ptr(), [16], dz.data_ptr(), dev.stream)
    assert np.array_equal(dev.download(dz)[: 16 * n].view(np.uint64), want.view(np.uint64)), "conj"
    cpu.binary("multiply", "cdouble", [n], [16], a.ctypes.data, [16], b.ctypes.data, [16], want.ctypes.data)
    gpu.binary("multiply", "cdouble", [n], [16], da.data_ptr(), [16], db.data_ptr(), [16], dz.data_ptr(), dev.stream)
    assert np.array_equal(dev.download(dz)[: 16 * n].view(np.uint64), want.view(np.uint64)), "multiply"
    wabs = np.empty(n, dtype=np.float64)
    cpu.unary("absolute", "cdouble", [n], [16], a.ctypes.data, [8], wabs.ctypes.data)
    gpu.unary("absolute", "cdouble", [n], [16], da.data_ptr(), [8], dz.data_ptr(), dev.stream)
    dist = util.ulp_distance(dev.download(dz)[: 8 * n].view(np.float64), wabs, "double")
    assert int(dist.max()) <= 2, "absolute: %d ulp" % int(dist.max())


def test_c4_half_axpy_2p26(gpu, cpu_all):
    cpu = cpu_all
    dev = util.Device()
    n = 1 << 26
    x = util.f32_to_solid_half(gen(0xC4C0).uniform(-4, 4, n).astype(np.float32))
    y = util.f32_to_solid_half(gen(0xC4C1).uniform(-4, 4, n).astype(np.float32))
    a = util.f32_to_solid_half(np.array([0.5], dtype=np.float32))
    t, want = np.empty(n, dtype=np.uint16), np.empty(n, dtype=np.uint16)
    cpu.binary("multiply", "half", [n], [2], x.ctypes.data, [0], a.ctypes.data, [2], t.ctypes.data)
    cpu.binary("add", "half", [n], [2], t.ctypes.data, [2], y.ctypes.data, [2], want.ctypes.data)
    dx, dy, dz = dev.upload(raw(x)), dev.upload(raw(y)), dev.empty(2 * n)
    gpu.axpy("half", [n], a.tobytes(), [2], dx.data_ptr(), [2], dy.data_ptr(), [2], dz.data_ptr(), dev.stream)
    assert np.array_equal(dev.download(dz)[: 2 * n].view(np.uint16), want)


# ---------------------------------------------------------------------------------------------------------------
def c5_constants(log2n):
    return json.loads((GOLDEN / "c5_constants.json").read_text())[str(log2n)]


def check_c5_sums(got_sum, got_sumsq, n, truth_sum, truth_sumsq, truth_sum_abs, what):
    """Deterministic bound of util.accumulation_bound on both sums, and on the signed sum the statistical bound for
    data with random signs: the rounding error of a tree over n such terms has standard deviation about
    u sqrt(n log2 n) rms(z); 16 of those are allowed (at n = 2^32: 0.36, where dropping 1 % of the elements moves
    the sum by about 4000)."""
    util.assert_accumulation(np.float64(got_sum), truth_sum, n, "float", truth_sum_abs, what + " sum")
    util.assert_accumulation(np.float64(got_sumsq), truth_sumsq, n, "float", truth_sumsq, what + " sum of squares")
    stat = 16 * 2.0 ** -24 * np.sqrt(n * np.log2(n)) * np.sqrt(truth_sumsq / n)
    assert abs(float(got_sum) - truth_sum) <= stat, "%s sum: %r against %r, statistical bound %g" % (what, got_sum, truth_sum, stat)


def test_c5_shard_2p28_against_reference(gpu, cpu_all):
    """A 2^28-element shard of the headline step (what one of 16 ranks would own): z bit-exact with the reference's multiply-then-add, the two
    sums against the reference's sum / norm2 of z and against the committed float64 constants."""
    cpu = cpu_all
    import bench
    dev = util.Device()
    n = 1 << 28
    x, y = bench.hash_uniform_numpy(0, n, 1), bench.hash_uniform_numpy(0, n, 2)
    a = np.array([0.5], dtype=np.float32)
    t, z = np.empty_like(x), np.empty_like(x)
    cpu.binary("multiply", "float", [n], [4], x.ctypes.data, [0], a.ctypes.data, [4], t.ctypes.data)
    cpu.binary("add", "float", [n], [4], t.ctypes.data, [4], y.ctypes.data, [4], z.ctypes.data)
    s_ref = scalar(cpu.reduce_all("sum", "float", [n], [4], z.ctypes.data), "float")
    q_ref = scalar(cpu.reduce_all("norm2", "float", [n], [4], z.ctypes.data), "float")
    dx, dy, dz = dev.upload(raw(x)), dev.upload(raw(y)), dev.empty(4 * n)
    part = dev.empty(gpu.axpy_sums_buffer_size(0, n))
    sums = dev.empty(8)
    gpu.axpy_sums("float", n, a.tobytes(), dx.data_ptr(), dy.data_ptr(), dz.data_ptr(), sums.data_ptr(), part.data_ptr(), dev.stream)
    assert np.array_equal(dev.download(dz)[: 4 * n].view(np.uint32), z.view(np.uint32)), "z"
    got = dev.download(sums)[:8].view(np.float32)
    c = c5_constants(28)
    check_c5_sums(got[0], got[1], n, c["sum"], c["sumsq"], c["sum_abs"], "C5 2^28")
    assert abs(float(got[0]) - float(s_ref)) <= 1e-5 * np.sqrt(n) * c["sum_abs"]
    assert abs(np.sqrt(float(got[1])) - float(q_ref)) <= 1e-5 * np.sqrt(n) * c["norm2"]
    # the host data really is the hashed sequence the constants were made from
    assert abs(float(z.astype(np.float64).sum()) - c["sum"]) <= 1e-9 * c["sum_abs"]


def test_c5_full_2p32_against_float64_constants(gpu):
    """The whole 2^32-element workload on one GPU (48 GiB) against float64 sums computed on the host by
    tests/golden/make_c5_constants.py from the same counter hash."""
    import torch
    import bench
    n = 1 << 32
    free, _ = torch.cuda.mem_get_info()
    if free < 52 * 2 ** 30:
        pytest.skip("needs 48 GiB of device memory")
    c = c5_constants(32)
    x = torch.empty(n, dtype=torch.float32, device="cuda")
    y = torch.empty(n, dtype=torch.float32, device="cuda")
    z = torch.empty(n, dtype=torch.float32, device="cuda")
    bench.hash_uniform_torch(0, n, 1, x)
    bench.hash_uniform_torch(0, n, 2, y)
    part = torch.empty(gpu.axpy_sums_buffer_size(0, n), dtype=torch.uint8, device="cuda")
    sums = torch.zeros(2, dtype=torch.float32, device="cuda")
    a = np.array([0.5], dtype=np.float32)
    gpu.axpy_sums("float", n, a.tobytes(), x.data_ptr(), y.data_ptr(), z.data_ptr(), sums.data_ptr(), part.data_ptr(),
                  torch.cuda.current_stream().cuda_stream)
    got = sums.cpu().numpy()
    check_c5_sums(got[0], got[1], n, c["sum"], c["sumsq"], c["sum_abs"], "C5 2^32")
    assert abs(np.sqrt(float(got[1])) - c["norm2"]) <= 2.0 ** -23 * c["norm2"] * 2, "norm2 within 2 float ulp"
    # z itself, spot-checked against the host evaluation of the same hash on windows at both ends and across the
    # 2^31 and 3 * 2^30 element marks (where 32-bit element counts or byte offsets would wrap)
    w = 1 << 20
    for start in (0, (1 << 30) - w // 2, (1 << 31) - w // 2, 3 * (1 << 30) - w // 2, n - w):
        hx, hy = bench.hash_uniform_numpy(start, w, 1), bench.hash_uniform_numpy(start, w, 2)
        want = (np.float32(0.5) * hx + hy).astype(np.float32)
        assert np.array_equal(z[start: start + w].cpu().numpy().view(np.uint32), want.view(np.uint32)), start
    del x, y, z, part
    torch.cuda.empty_cache()
