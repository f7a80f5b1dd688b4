"""Parity of the copy/convert/byteswap family with the reference's Solid CPU library
(solid_cpu_copy[T1][T2], solid_cpu_byteswap_copy[T1][T2], solid_cpu_byteswap[T]).
Every result is compared bit for bit: conversions, byte reversal and the
reference's own half rounding are exact operations.

Floating-point sources converted to integer types stay inside the range of the
destination: out-of-range float->int casts are undefined behaviour in the
reference's C code and are not part of the contract.
"""
import numpy as np
import pytest

import util
from solid_b200 import dtypes as dt

pytestmark = pytest.mark.gpu


def source_kind(src, dst):
    if dst in dt.UINT or dst == "bool":
        return "positive" if src in dt.GROUPS["float"] or src in dt.SINT else "general"
    return "general"


def run_pair(gpu, cpu, dev, src, dst, size1, v1, size2, v2, rng, variant="copy", kind=None):
    a = util.fill_buffer(v1, rng, kind or source_kind(src, dst))
    if variant == "byteswap_copy":                      # store the source with reversed bytes
        a = swap_buffer(a, src, v1)
    d0 = util.fill_buffer(v2, rng, "general")
    want = d0.copy()
    cpu.copy(src, dst, size1, v1.strides, a.ctypes.data + v1.offset, size2, v2.strides,
             want.ctypes.data + v2.offset, variant=variant)
    da, dd = dev.upload(a), dev.upload(d0)
    gpu.copy(src, dst, size1, v1.strides, da.data_ptr() + v1.offset, size2, v2.strides,
             dd.data_ptr() + v2.offset, dev.stream, variant=variant)
    got = dev.download(dd)
    assert np.array_equal(got, want), "%s %s->%s sizes %s %s" % (variant, src, dst, size1, size2)


def swap_buffer(buf, dtype, view):
    """Reverse the bytes of every real component of every (aligned-grid) element of the buffer."""
    comp = dt.SIZE[dt.elem_type(dtype)]
    head = view.offset % dt.SIZE[dtype]
    body = buf[head: head + ((len(buf) - head) // comp) * comp].reshape(-1, comp)[:, ::-1].reshape(-1)
    out = buf.copy()
    out[head: head + len(body)] = body
    return out


@pytest.mark.parametrize("src", dt.NAMES)
def test_copy_all_pairs(src, gpu, cpu):
    dev = util.Device()
    rng = np.random.default_rng(100 + dt.INDEX[src])
    for dst in dt.NAMES:
        # contiguous, ragged length
        n = 4099
        run_pair(gpu, cpu, dev, src, dst, [n], util.dense_view(src, [n]), [n], util.dense_view(dst, [n]), rng)
        # padded source, transposed destination
        v1 = util.dense_view(src, [33, 21], pad_elems=5)
        vd = util.dense_view(dst, [21, 33]); v2 = util.View(dst, [33, 21], [vd.strides[1], vd.strides[0]], 0, vd.nbytes)
        run_pair(gpu, cpu, dev, src, dst, [33, 21], v1, [33, 21], v2, rng)
        # different shapes, equal element count
        run_pair(gpu, cpu, dev, src, dst, [12, 10], util.dense_view(src, [12, 10], pad_elems=2),
                 [8, 5, 3], util.dense_view(dst, [8, 5, 3], pad_elems=1), rng)
        # regular entry point and empty tensors
        run_pair(gpu, cpu, dev, src, dst, [0], util.dense_view(src, [0]), [0], util.dense_view(dst, [0]), rng)


@pytest.mark.parametrize("src", dt.NAMES)
def test_byteswap_copy_all_pairs(src, gpu, cpu):
    dev = util.Device()
    rng = np.random.default_rng(200 + dt.INDEX[src])
    for dst in dt.NAMES:
        n = 1031
        run_pair(gpu, cpu, dev, src, dst, [n], util.dense_view(src, [n]), [n], util.dense_view(dst, [n]), rng,
                 variant="byteswap_copy")
        run_pair(gpu, cpu, dev, src, dst, [16, 9], util.dense_view(src, [16, 9], pad_elems=4),
                 [9, 16], util.dense_view(dst, [9, 16]), rng, variant="byteswap_copy")


@pytest.mark.parametrize("dtype", dt.NAMES)
def test_byteswap_in_place(dtype, gpu, cpu):
    dev = util.Device()
    rng = np.random.default_rng(300 + dt.INDEX[dtype])
    for size, pad in (([4099], 0), ([17, 9], 3), ([], 0), ([0], 0)):
        v = util.dense_view(dtype, size, pad_elems=pad)
        buf = util.fill_buffer(v, rng)
        want = buf.copy()
        cpu.byteswap(dtype, size, v.strides, want.ctypes.data)
        d = dev.upload(buf)
        gpu.byteswap(dtype, size, v.strides, d.data_ptr(), dev.stream)
        assert np.array_equal(dev.download(d), want), "byteswap_%s %s" % (dtype, size)


UNALIGNED_PAIRS = [("double", "half"), ("double", "float"), ("float", "double"), ("int32", "double"),
                   ("int64", "int16"), ("cdouble", "cfloat"), ("uint16", "uint16"), ("half", "float"),
                   ("cfloat", "bool"), ("double", "double"), ("uint32", "half"), ("chalf", "cdouble")]


@pytest.mark.parametrize("src,dst", UNALIGNED_PAIRS)
def test_unaligned_and_byteswapped(src, dst, gpu, cpu):
    """Source and/or destination start at byte offsets that are not multiples of the element
    size (3 bytes for the source, 1 for the destination), with and without reversed source bytes."""
    dev = util.Device()
    rng = np.random.default_rng(7)
    es, ed = dt.SIZE[src], dt.SIZE[dst]
    for n in (1, 5, 4099):
        for soff, doff in ((3, 0), (0, 1), (3, 1), (es + 1, 0)):
            if (es == 1 and soff % es == 0 and doff % ed == 0):
                continue
            v1 = util.View(src, [n], [es], soff, n * es + soff + 64)
            v2 = util.View(dst, [n], [ed], doff, n * ed + doff + 64)
            for variant in ("copy", "byteswap_copy"):
                run_pair(gpu, cpu, dev, src, dst, [n], v1, [n], v2, rng, variant=variant)
    # strided unaligned: rows of 37 elements, 3 bytes of padding per row
    v1 = util.View(src, [37, 11], [es, 37 * es + 3], 3, 11 * (37 * es + 3) + 64)
    v2 = util.dense_view(dst, [37, 11])
    run_pair(gpu, cpu, dev, src, dst, [37, 11], v1, [37, 11], v2, rng, variant="byteswap_copy")


def test_copy_ex_destination_swapped(gpu, cpu):
    """copy_ex with both byte orders: oracle = byteswap_copy followed by an in-place byteswap of the result."""
    dev = util.Device()
    rng = np.random.default_rng(11)
    for src, dst in (("int32", "double"), ("double", "half"), ("float", "cfloat"), ("int16", "int64")):
        n = 2053
        v1, v2 = util.dense_view(src, [n]), util.dense_view(dst, [n])
        a = swap_buffer(util.fill_buffer(v1, rng), src, v1)
        d0 = np.zeros(v2.nbytes, dtype=np.uint8)
        want = d0.copy()
        cpu.copy(src, dst, [n], v1.strides, a.ctypes.data, [n], v2.strides, want.ctypes.data, variant="byteswap_copy")
        cpu.byteswap(dst, [n], v2.strides, want.ctypes.data)
        da, dd = dev.upload(a), dev.upload(d0)
        gpu.copy_ex(src, dst, 3, [n], v1.strides, da.data_ptr(), [n], v2.strides, dd.data_ptr(), dev.stream)
        assert np.array_equal(dev.download(dd), want), "copy_ex %s->%s" % (src, dst)
