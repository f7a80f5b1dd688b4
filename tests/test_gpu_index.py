"""Parity of the indexed-access entry points with the reference's Solid CPU library
(solid/src/core/cpu/template_index.c): get_index, set_index, fill_index with per-dimension tables
of byte offsets (or plain strides), add_if_negative and index_to_offset.  Everything is bit-exact;
the tables of the scatter cases hold distinct positions (duplicates make the reference
order-dependent too), the fill cases repeat positions on purpose.
"""
import numpy as np
import pytest

import util
from solid_b200 import dtypes as dt
from solid_b200 import oplist as ol

pytestmark = pytest.mark.gpu


def index_cases(dtype, rng):
    """(name, size of the selection, offsets tables (numpy int64 or None), strides1, source shape)."""
    es = dt.SIZE[dtype]
    cases = []
    # vector gather: 1-D table
    src = [1000]
    cases.append(("vector", [257], [rng.permutation(1000)[:257].astype(np.int64) * es], [0], src))
    # rows picked by a table, columns by stride (column-major source 40 x 30)
    src = [40, 30]
    cases.append(("rows", [17, 30], [rng.permutation(40)[:17].astype(np.int64) * es, None], [0, 40 * es], src))
    # both dimensions through tables
    cases.append(("rows_cols", [9, 11], [rng.permutation(40)[:9].astype(np.int64) * es,
                                          rng.permutation(30)[:11].astype(np.int64) * 40 * es], [0, 0], src))
    # three dimensions, the middle one through a table, reversed order along it
    src = [6, 20, 5]
    cases.append(("middle", [6, 13, 5], [None, np.sort(rng.permutation(20)[:13])[::-1].astype(np.int64) * 6 * es, None],
                  [es, 0, 120 * es], src))
    # no table at all (plain strided copy) and an empty selection
    cases.append(("strided", [8, 7], [None, None], [es, 40 * es], [40, 30]))
    cases.append(("empty", [0, 30], [np.zeros(0, dtype=np.int64), None], [0, 40 * es], [40, 30]))
    cases.append(("scalar", [], [], [], [3]))
    # whole runs along dimension 0 (no table there, at least 1 KB long): columns picked by a table; the second case
    # has runs of more than one 16 KB piece for the wider types and starts that are not 16-byte aligned
    src = [1100, 20]
    cases.append(("runs", [1100, 13], [None, rng.permutation(20)[:13].astype(np.int64) * 1100 * es], [es, 0], src))
    src = [5003, 9]
    cases.append(("long_runs", [5003, 5], [None, rng.permutation(9)[:5].astype(np.int64) * 5003 * es], [es, 0], src))
    src = [1030, 3, 6]
    cases.append(("runs_3d", [1030, 3, 4], [None, None, rng.permutation(6)[:4].astype(np.int64) * 3090 * es],
                  [es, 1030 * es, 0], src))
    # gathers along dimension 0 into a destination that is contiguous there: a span that fits the shared-memory
    # window (any alignment of its first byte), one that does not (for elements of 2 bytes and more), and a long 1-d one
    src = [400, 7]
    cases.append(("gather0", [300, 7], [rng.permutation(400)[:300].astype(np.int64) * es, None], [0, 400 * es], src))
    src = [40000, 3]
    cases.append(("gather0_wide", [300, 3], [np.sort(rng.permutation(40000)[:300]).astype(np.int64) * es, None], [0, 40000 * es], src))
    src = [9000]
    cases.append(("gather0_1d", [8500], [(rng.permutation(9000)[:8500].astype(np.int64)) * es], [0], src))
    return cases


def run_tables(dev, tables):
    """Upload offset tables; returns (device tensors to keep alive, device addresses, host addresses)."""
    keep, daddr, haddr = [], [], []
    for t in tables:
        if t is None:
            daddr.append(None); haddr.append(None)
        else:
            t = np.ascontiguousarray(t)
            d = dev.upload(t.view(np.uint8)) if t.size else dev.empty(16)
            keep.append((t, d)); daddr.append(d.data_ptr()); haddr.append(t.ctypes.data if t.size else None)
    return keep, daddr, haddr


@pytest.mark.parametrize("dtype", dt.NAMES)
def test_get_set_fill_index_match_reference(dtype, gpu, cpu):
    dev = util.Device()
    rng = np.random.default_rng(300 + dt.INDEX[dtype])
    es = dt.SIZE[dtype]
    for name, size, tables, strides1, srcshape in index_cases(dtype, rng):
        vsrc = util.dense_view(dtype, srcshape)
        vsel = util.dense_view(dtype, size, pad_elems=2 if len(size) > 1 else 0)
        keep, daddr, haddr = run_tables(dev, tables)
        if name == "empty":
            haddr[0] = keep[0][0].ctypes.data if keep[0][0].size else haddr[0]
        a = util.fill_buffer(vsrc, rng, "general")
        b = util.fill_buffer(vsel, rng, "general")
        # get: selection <- indexed source
        want = b.copy()
        cpu.index2("get_index", dtype, size, haddr, strides1, a.ctypes.data, vsel.strides, want.ctypes.data + vsel.offset)
        da, db = dev.upload(a), dev.upload(b)
        gpu.index2("get_index", dtype, size, daddr, strides1, da.data_ptr(), vsel.strides, db.data_ptr() + vsel.offset, dev.stream)
        assert np.array_equal(dev.download(db), want), ("get_index", dtype, name)
        # set: indexed source <- selection (distinct positions)
        want = a.copy()
        cpu.index2("set_index", dtype, size, haddr, strides1, want.ctypes.data, vsel.strides, b.ctypes.data + vsel.offset)
        da, db = dev.upload(a), dev.upload(b)
        gpu.index2("set_index", dtype, size, daddr, strides1, da.data_ptr(), vsel.strides, db.data_ptr() + vsel.offset, dev.stream)
        assert np.array_equal(dev.download(da), want), ("set_index", dtype, name)
        # fill
        value = util.random_values(dtype, 1, rng, "general").view(np.uint8)[:es].tobytes()
        want = a.copy()
        cpu.fill_index(dtype, size, haddr, strides1, want.ctypes.data, value)
        da = dev.upload(a)
        gpu.fill_index(dtype, size, daddr, strides1, da.data_ptr(), value, dev.stream)
        assert np.array_equal(dev.download(da), want), ("fill_index", dtype, name)
    # fill through a table with repeated positions
    tab = (rng.integers(0, 50, 400).astype(np.int64)) * es
    keep, daddr, haddr = run_tables(dev, [tab])
    v = util.dense_view(dtype, [50])
    a = util.fill_buffer(v, rng, "general")
    value = util.random_values(dtype, 1, rng, "general").view(np.uint8)[:es].tobytes()
    want = a.copy()
    cpu.fill_index(dtype, [400], haddr, [0], want.ctypes.data, value)
    da = dev.upload(a)
    gpu.fill_index(dtype, [400], daddr, [0], da.data_ptr(), value, dev.stream)
    assert np.array_equal(dev.download(da), want), ("fill_index repeated", dtype)


@pytest.mark.parametrize("dtype", dt.GROUPS[ol.INDEX_OPS["add_if_negative"]])
def test_add_if_negative_matches_reference(dtype, gpu, cpu):
    dev = util.Device()
    rng = np.random.default_rng(7)
    npdt = dt.NUMPY[dtype]
    for size, pad in (([1000], 0), ([33, 9], 5), ([], 0), ([0], 0)):
        v = util.dense_view(dtype, size, pad_elems=pad)
        buf = np.zeros(v.nbytes, dtype=np.uint8)
        vals = rng.integers(-50, 50, v.nbytes // dt.SIZE[dtype]).astype(npdt)
        buf[: vals.nbytes] = vals.view(np.uint8)
        value = np.array([50], dtype=npdt).tobytes()
        want = buf.copy()
        cpu.add_if_negative(dtype, size, v.strides, want.ctypes.data + v.offset, value)
        d = dev.upload(buf)
        gpu.add_if_negative(dtype, size, v.strides, d.data_ptr() + v.offset, value, dev.stream)
        assert np.array_equal(dev.download(d), want), (dtype, size)


@pytest.mark.parametrize("dtype", dt.GROUPS[ol.INDEX_OPS["index_to_offset"]])
def test_index_to_offset_matches_reference(dtype, gpu, cpu):
    dev = util.Device()
    rng = np.random.default_rng(11)
    npdt = dt.NUMPY[dtype]; es = dt.SIZE[dtype]
    for nstr, nelem, layout in ((3, 500, "tuples"), (1, 77, "tuples"), (4, 129, "planes"), (2, 0, "tuples")):
        strides = [int(s) for s in rng.integers(-64, 4096, nstr)]
        idx = rng.integers(0, 100, (nstr, max(nelem, 1))).astype(npdt)         # idx[i, e]
        if layout == "tuples":      # the components of one tuple are adjacent: column-major nstr x nelem
            host = np.asfortranarray(idx); stride_reduce, stride1 = es, nstr * es
        else:                       # one plane per component: column-major nelem x nstr
            host = np.ascontiguousarray(idx); stride_reduce, stride1 = max(nelem, 1) * es, es
        raw = host.reshape(-1, order="A").view(np.uint8).copy()
        want = np.full(max(nelem, 1) * 2, -1, dtype=np.int64)                  # destination stride 16: every other slot
        got0 = want.copy()
        cpu.index_to_offset(dtype, strides, stride_reduce, nelem, stride1, raw.ctypes.data, 16, want.ctypes.data)
        d_in, d_out = dev.upload(raw), dev.upload(got0.view(np.uint8))
        gpu.index_to_offset(dtype, strides, stride_reduce, nelem, stride1, d_in.data_ptr(), 16, d_out.data_ptr(), dev.stream)
        assert np.array_equal(dev.download(d_out).view(np.int64)[: want.size], want), (dtype, nstr, nelem, layout)
