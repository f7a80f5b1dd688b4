"""The Ocean-level dispatch library (include/ocean_gpu_b200.h): exported symbols, the error
behaviour of the reference's dispatch functions (typed "not supported" errors from table holes,
precondition checks) without a GPU, and on the GPU the stream protocol, the scratch cache and the
host-scalar results."""
import ctypes as C
import re
import subprocess
from pathlib import Path

import numpy as np
import pytest

import util

from solid_b200 import _ocean, dtypes as dt, oplist as ol
from solid_b200._ocean import OceanError, TensorView

ROOT = Path(__file__).resolve().parent.parent


def fake_view(dtype="float", size=(4,), device=0, byteswapped=False):
    v = TensorView()
    v.dtype, v.ndims = dt.INDEX[dtype], len(size)
    step = dt.SIZE[dtype]
    for i, s in enumerate(size):
        v.size[i], v.strides[i] = s, step
        step *= s
    v.data, v.device, v.byteswapped = 256, device, int(byteswapped)
    return v


def test_dispatch_library_exports_declared_functions():
    out = subprocess.run(["gcc", "-E", "-P", "-I", str(ROOT / "include"), "-I", "/usr/local/cuda/include",
                          str(ROOT / "include" / "ocean_gpu_b200.h")], stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)
    assert out.returncode == 0, out.stderr[-1500:]
    names = set(re.findall(r"\b(OcTensorGPU_\w+|OcGPU_\w+|OcInitGPU_B200|OcFinalizeGPU_B200)\s*\(", out.stdout))
    assert len(names) > 120
    oc = _ocean.get()
    missing = sorted(n for n in names if not hasattr(oc.dll, n))
    assert not missing, missing
    # every Solid operation of the path is reachable under its Ocean name
    for fam in (ol.UNARY_OPS, ol.BINARY_OPS, ol.REDUCE_BOOL_OPS, ol.REDUCE_BOUND1_OPS, ol.REDUCE_BOUND2_OPS,
                ol.REDUCE_U64_OPS, ol.REDUCE_VOID_OPS, ol.REDUCE_NORM_OPS, ol.AXIS_OPS, ol.AXIS_NORM_OPS):
        for n in fam:
            assert oc.has(_ocean.ocean_name(n)), n


def test_name_mapping():
    assert _ocean.ocean_name("multiply") == "scale"
    assert _ocean.ocean_name("bitwise_not") == "bitwiseNot"
    assert _ocean.ocean_name("true_divide") == "trueDivide"
    assert _ocean.ocean_name("lt") == "elemwiseLT"
    assert _ocean.ocean_name("sum_abs_nan") == "sumAbsNaN"
    assert _ocean.ocean_name("all_gtle") == "allGTLE"
    assert _ocean.ocean_name("axis_norm2_nan") == "axisNorm2NaN"
    assert _ocean.ocean_name("any_inf") == "anyInf"


def test_reduction_result_types_agree_with_python_table():
    oc = _ocean.get()
    for op in list(ol.REDUCE_BOOL_OPS) + list(ol.REDUCE_U64_OPS) + list(ol.REDUCE_VOID_OPS) + list(ol.REDUCE_NORM_OPS):
        for t in dt.NAMES:
            assert oc.result_type(op, t) == ol.reduce_result_type(op, t), (op, t)
            assert oc.result_type("axis_" + op, t) == ol.reduce_result_type(op, t)


def test_errors_before_any_cuda_call():
    oc = _ocean.get()
    a, b, d = fake_view("float"), fake_view("float"), fake_view("float")
    with pytest.raises(OceanError, match="not available for type bool"):
        vb = fake_view("bool")
        oc._check(oc.fn("sin")(C.byref(vb), C.byref(vb)), "sin")
    with pytest.raises(OceanError, match="not available for type float"):
        oc._check(oc.fn("bitwiseAnd")(C.byref(a), C.byref(b), C.byref(d)), "bitwiseAnd")
    with pytest.raises(OceanError, match="not available for type complex-double"):
        vc = fake_view("cdouble")
        oc._check(oc.fn("floorDivide")(C.byref(vc), C.byref(vc), C.byref(vc)), "floorDivide")
    with pytest.raises(OceanError, match="size mismatch"):
        other = fake_view("float", (5,))
        oc._check(oc.fn("add")(C.byref(a), C.byref(other), C.byref(d)), "add")
    with pytest.raises(OceanError, match="native byte order"):
        sw = fake_view("float", byteswapped=True)
        oc._check(oc.fn("add")(C.byref(sw), C.byref(b), C.byref(d)), "add")
    with pytest.raises(OceanError, match="number of elements"):
        oc._check(oc.fn("copy")(C.byref(a), C.byref(fake_view("double", (3,)))), "copy")
    with pytest.raises(OceanError, match="must have type"):
        ax = (C.c_int * 1)(0)
        m = fake_view("float", (4, 3)); o = fake_view("double", (3,))
        oc._check(oc.fn("axisSum")(C.byref(m), C.c_int(1), ax, C.byref(o)), "axisSum")
    with pytest.raises(OceanError, match="out of range"):
        ax = (C.c_int * 1)(7)
        m = fake_view("float", (4, 3)); o = fake_view("float", (3,))
        oc._check(oc.fn("axisSum")(C.byref(m), C.c_int(1), ax, C.byref(o)), "axisSum")
    with pytest.raises(OceanError, match="data type of the tensor"):
        sv = oc.scalar(b"\0" * 8, "double")
        oc._check(oc.fn("fill")(C.byref(a), C.byref(sv)), "fill")
    # operand and result types: the kernel is chosen by the first operand and would read or write the others as
    # the types it expects, past the end of a narrower buffer
    with pytest.raises(OceanError, match="destination of sqrt on type float must have type float, not int8"):
        oc._check(oc.fn("sqrt")(C.byref(a), C.byref(fake_view("int8"))), "sqrt")
    with pytest.raises(OceanError, match="must have type bool, not float"):
        oc._check(oc.fn("isnan")(C.byref(a), C.byref(d)), "isnan")
    with pytest.raises(OceanError, match="must have type double, not complex-double"):
        vc = fake_view("cdouble")
        oc._check(oc.fn("absolute")(C.byref(vc), C.byref(vc)), "absolute")
    with pytest.raises(OceanError, match="second operand of add on type float must have type float, not double"):
        oc._check(oc.fn("add")(C.byref(a), C.byref(fake_view("double")), C.byref(d)), "add")
    with pytest.raises(OceanError, match="destination of add on type float must have type float, not half"):
        oc._check(oc.fn("add")(C.byref(a), C.byref(b), C.byref(fake_view("half"))), "add")
    with pytest.raises(OceanError, match="must have type bool, not float"):
        oc._check(oc.fn("elemwiseLT")(C.byref(a), C.byref(b), C.byref(d)), "elemwiseLT")
    i32, u32 = fake_view("int32"), fake_view("uint32")
    with pytest.raises(OceanError, match="second operand of bitshiftLeft on type int32 must have type int8"):
        oc._check(oc.fn("bitshiftLeft")(C.byref(i32), C.byref(i32), C.byref(i32)), "bitshiftLeft")
    with pytest.raises(OceanError, match="destination of bitshiftLeft"):
        oc._check(oc.fn("bitshiftLeft")(C.byref(i32), C.byref(fake_view("int8")), C.byref(fake_view("int16"))), "bitshiftLeft")
    with pytest.raises(OceanError, match="second operand of power on type int32 must have type int16"):
        oc._check(oc.fn("power")(C.byref(i32), C.byref(i32), C.byref(i32)), "power")
    with pytest.raises(OceanError, match="on the device of the destination"):
        oc._check(oc.fn("add")(C.byref(a), C.byref(fake_view("float", device=1)), C.byref(d)), "add")
    with pytest.raises(OceanError, match="on the device of the destination"):
        oc._check(oc.fn("negative")(C.byref(fake_view("float", device=1)), C.byref(d)), "negative")


# ------------------------------------------------------------------------------------ GPU
@pytest.mark.gpu
def test_results_and_scratch_cache_rotation(gpu):
    """Many host-returning reductions in a row (the scratch cache has three slots) with sizes that
    force the slots to grow, checked against float64 sums."""
    from solid_b200 import Tensor, ops
    _ocean.get().init()
    rng = np.random.default_rng(1)
    for n in (10, 100000, 5, 3000000, 17, 1 << 22, 1000):
        x = rng.uniform(-1, 1, n).astype(np.float32)
        t = Tensor.from_numpy(x)
        assert abs(float(ops.sum(t)) - x.astype(np.float64).sum()) <= util.accumulation_bound(n, "float", np.abs(x).sum())
        assert ops.maximum(t) == x.max() and ops.nnz(t) == np.count_nonzero(x)
        assert ops.all(t) == np.uint8(np.all(x != 0))
        assert ops.reduce_all("all_gtlt", t, bounds=(-1.5, 1.5)) == 1
        assert ops.reduce_all("all_lt", t, bounds=(0.0,)) == 0 or n < 20
    m = rng.normal(size=(300, 200))
    tm = Tensor.from_numpy(m)
    assert np.allclose(ops.sum(tm, 0).numpy(), m.sum(axis=0), atol=1e-9)
    assert np.allclose(ops.norm(tm, 3, [1]).numpy(), (np.abs(m) ** 3).sum(axis=1) ** (1 / 3), rtol=1e-5)


@pytest.mark.gpu
def test_scalar_forms_equal_tensor_forms(gpu):
    """OcTensorGPU_addScalar and relatives (scalar by value) against the tensor operation with a 0-d operand,
    which is how the reference runs them; also into a transposed destination and with a mismatched scalar type."""
    from solid_b200 import Tensor, ops, dtypes as dt
    import ctypes as C
    _ocean.get().init()
    rng = np.random.default_rng(5)
    x = rng.normal(size=(37, 11)).astype(np.float32)
    t = Tensor.from_numpy(np.asfortranarray(x))
    s0 = Tensor.from_numpy(np.array(1.75, dtype=np.float32))
    for name, fn in (("add", ops.add), ("subtract", ops.subtract), ("multiply", ops.scale)):
        assert np.array_equal(ops.scalar_op(name, t, 1.75).numpy(), fn(t, s0).numpy()), name
    k = rng.integers(-1000, 1000, 501).astype(np.int16)
    tk = Tensor.from_numpy(k)
    for name, ref in (("bitwise_and", k & 0x0F0F), ("bitwise_or", k | 0x0F0F), ("bitwise_xor", k ^ 0x0F0F)):
        assert np.array_equal(ops.scalar_op(name, tk, 0x0F0F).numpy(), ref), name
    out = Tensor.empty([11, 37], "float").T
    ops.scalar_op("multiply", t, -2.0, out)
    assert np.array_equal(out.numpy(), x * np.float32(-2.0))
    with pytest.raises(TypeError):
        ops.scalar_op("bitwise_and", t, 3)
    oc = _ocean.get()
    bad = oc.scalar(b"\0" * 8, "double")
    v = oc.view(t, 0)
    with pytest.raises(_ocean.OceanError, match="type mismatch"):
        oc._check(oc.fn("addScalar")(C.byref(v), C.byref(bad), C.byref(v)), "addScalar")


@pytest.mark.gpu
def test_ranges_count_in_memory_order(gpu):
    """OcTensorGPU_steps* reduce the tensor to its memory layout first, as the reference's dispatch does: a
    matrix, its transpose and a view with a reversed dimension over the same bytes all receive the same values."""
    from solid_b200 import Tensor
    import ctypes as C
    oc = _ocean.get(); oc.init()
    t = Tensor.empty([12, 7], "float")
    views = [t, t.T, t.as_strided([12, 7], [-4, 48], offset=44)]
    want = (2.5 + 0.25 * np.arange(84)).astype(np.float32)
    for v in views:
        t.storage.zero_()
        tv = oc.view(v, 0)
        oc._check(oc.fn("stepsDouble")(C.byref(tv), C.c_double(2.5), C.c_double(0.25)), "stepsDouble")
        assert np.array_equal(t.numpy().reshape(-1, order="F"), want)
    k = Tensor.empty([5, 4], "int16")
    kv = oc.view(k, 0)
    oc._check(oc.fn("stepsInt64")(C.byref(kv), C.c_int64(-3), C.c_int64(2)), "stepsInt64")
    assert np.array_equal(k.numpy().reshape(-1, order="F"), (-3 + 2 * np.arange(20)).astype(np.int16))
    with pytest.raises(_ocean.OceanError, match="not available for type"):
        from solid_b200._lib import CDouble
        oc._check(oc.fn("stepsCDouble")(C.byref(kv), CDouble(0, 0), CDouble(1, 0)), "stepsCDouble")


@pytest.mark.gpu
def test_indexed_access_through_the_dispatch(gpu):
    """OcTensorGPU_getIndex / setIndex / fillIndex / addIfNegative / indexToOffset against numpy's outer indexing."""
    from solid_b200 import Tensor, ops
    import ctypes as C
    oc = _ocean.get(); oc.init()
    rng = np.random.default_rng(21)
    a = rng.normal(size=(40, 30, 5)).astype(np.float32)
    t = Tensor.from_numpy(a)
    rows = rng.permutation(40)[:17]; planes = np.array([4, -1, 0])
    got = ops.take(t, [rows, None, planes]).numpy()
    assert np.array_equal(got, a[np.ix_(rows, np.arange(30), planes % 5)])
    tt = t.T                                                    # a view with permuted strides
    got = ops.take(tt, [planes, None, rows]).numpy()
    assert np.array_equal(got, a.transpose(2, 1, 0)[np.ix_(planes % 5, np.arange(30), rows)])
    vals = rng.normal(size=(17, 30, 3)).astype(np.float32)
    ops.put(t, [rows, None, [4, 3, 0]], Tensor.from_numpy(vals))
    want = a.copy(); want[np.ix_(rows, np.arange(30), [4, 3, 0])] = vals
    assert np.array_equal(t.numpy(), want)
    ops.fill_at(t, [[0, 0, 39], [1, 1], None], -7.5)
    want[np.ix_([0, 39], [1], np.arange(5))] = -7.5
    assert np.array_equal(t.numpy(), want)
    with pytest.raises(IndexError):
        ops.take(t, [[40], None, None])
    # negative indices wrapped on the device, then turned into offsets
    idx = np.asfortranarray(np.array([[3, -1, 0, 39], [-30, 29, 5, -2]], dtype=np.int64))      # 2 x 4 index tuples
    ti = Tensor.from_numpy(idx)
    for d, n in enumerate((40, 30)):
        row = ti.slice(0, d, d + 1)
        sv = oc.scalar(np.int64(n).tobytes(), "int64")
        rv = oc.view(row, 0)
        oc._check(oc.fn("addIfNegative")(C.byref(rv), C.byref(sv)), "addIfNegative")
    off = Tensor.empty([4], "int64")
    strides = (C.c_int64 * 2)(4, 160)
    tv, ov = oc.view(ti, 0), oc.view(off, 0)
    oc._check(oc.fn("indexToOffset")(C.byref(tv), strides, C.byref(ov)), "indexToOffset")
    wrapped = np.where(idx < 0, idx + np.array([[40], [30]]), idx)
    assert np.array_equal(off.numpy(), 4 * wrapped[0] + 160 * wrapped[1])


@pytest.mark.gpu
def test_stream_protocol_orders_producer_and_consumer(gpu):
    """The source is produced on one stream, the operation runs on the destination's stream: the
    dispatch must wait for the source's event, and record the destination's."""
    import torch
    from solid_b200 import Tensor
    oc = _ocean.get()
    n = 1 << 24
    s1, s2 = torch.cuda.Stream(), torch.cuda.Stream()
    e1 = torch.cuda.Event(); e2 = torch.cuda.Event()
    a = Tensor.empty([n], "float"); b = Tensor.empty([n], "float"); c = Tensor.empty([n], "float")
    torch.cuda.synchronize()
    one = oc.scalar(np.float32(1.0).tobytes(), "float"); two = oc.scalar(np.float32(2.0).tobytes(), "float")
    va = oc.view(a, s1.cuda_stream, e1.cuda_event if hasattr(e1, "cuda_event") else 0)
    # torch events expose their handle only after a record; record once so the handle exists
    with torch.cuda.stream(s1):
        e1.record()
    with torch.cuda.stream(s2):
        e2.record()
    va = oc.view(a, s1.cuda_stream, e1.cuda_event); vb = oc.view(b, s1.cuda_stream, e1.cuda_event)
    vc = oc.view(c, s2.cuda_stream, e2.cuda_event)
    for _ in range(5):                                        # producers on stream 1
        oc._check(oc.fn("fill")(C.byref(va), C.byref(one)), "fill")
        oc._check(oc.fn("fill")(C.byref(vb), C.byref(two)), "fill")
    oc._check(oc.fn("add")(C.byref(va), C.byref(vb), C.byref(vc)), "add")      # consumer on stream 2
    e2.synchronize()                                         # the destination's event was recorded by the dispatch
    got = c.storage[: 4 * n].cpu().numpy().view(np.float32)
    assert np.all(got == 3.0)
    torch.cuda.synchronize()


@pytest.mark.gpu
def test_scratch_slots_are_ordered_across_streams(gpu):
    """Split axis reductions take their partial-result buffer from a three-slot cache per device, so the fourth
    request reuses the first slot.  Six such reductions alternate over two streams, the first stream held back by
    a long idle kernel: without an event per slot the later calls on the free stream would overwrite partials that
    the held-back calls have not folded yet."""
    import torch
    from solid_b200 import Tensor
    oc = _ocean.get()
    rng = np.random.default_rng(12)
    rows, cols = 64, 1 << 15                                   # few outputs, long strided range: split over blocks
    hosts = [rng.integers(-1000, 1000, (rows, cols)).astype(np.int32) for _ in range(6)]
    srcs = [Tensor.from_numpy(np.asfortranarray(h)) for h in hosts]
    outs = [Tensor.empty([rows], "int64") for _ in range(6)]
    streams = [torch.cuda.Stream(), torch.cuda.Stream()]
    events = [torch.cuda.Event(), torch.cuda.Event()]
    for st, ev in zip(streams, events):
        with torch.cuda.stream(st):
            ev.record()
    torch.cuda.synchronize()
    axes = (C.c_int * 1)(1)
    with torch.cuda.stream(streams[0]):
        torch.cuda._sleep(int(4e8))                            # roughly 0.2 s before stream 0 may start
    for k in range(6):
        st, ev = streams[k % 2], events[k % 2]
        vs, vd = oc.view(srcs[k], st.cuda_stream, ev.cuda_event), oc.view(outs[k], st.cuda_stream, ev.cuda_event)
        oc._check(oc.fn("axisSum")(C.byref(vs), C.c_int(1), axes, C.byref(vd)), "axisSum")
    torch.cuda.synchronize()
    for k in range(6):
        assert np.array_equal(outs[k].numpy(), hosts[k].astype(np.int64).sum(axis=1)), k


@pytest.mark.gpu
def test_copy_between_devices_through_dense_temporaries(gpu):
    """The staged path (dense temporary on each device and one peer copy) is what runs where a device cannot load
    a peer's memory; on machines whose GPUs all see each other it is reached by OCEAN_B200_FORCE_STAGED_COPY=1,
    which the library reads once, hence the child process."""
    import os
    import sys
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    env = dict(os.environ, OCEAN_B200_FORCE_STAGED_COPY="1")
    res = subprocess.run([sys.executable, "-m", "pytest", "-q", "-x", "-m", "gpu",
                          "%s::test_copy_between_devices" % Path(__file__).resolve()],
                         env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, cwd=str(ROOT))
    assert res.returncode == 0 and "1 passed" in res.stdout, res.stdout[-2000:]


@pytest.mark.gpu
def test_copy_between_devices(gpu):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from solid_b200 import Tensor, ops
    x = np.arange(100000, dtype=np.int32)
    src = Tensor.from_numpy(x, device="cuda:0")
    dst = Tensor.empty([100000], "double", device="cuda:1")
    ops.copy(src.slice(0, 99999, -1, -1), dst)               # reversed, converted, other device
    torch.cuda.synchronize(0); torch.cuda.synchronize(1)
    assert np.array_equal(dst.numpy(), x[::-1].astype(np.float64))
    # a transposed matrix, the other way round, then back into a padded destination: repeated so that a
    # missing ordering between the two devices' streams would show
    m = np.random.default_rng(3).normal(size=(300, 200)).astype(np.float32)
    on1 = Tensor.from_numpy(np.asfortranarray(m), device="cuda:1")
    for _ in range(4):
        on0 = Tensor.empty([200, 300], "double", device="cuda:0")
        ops.copy(on1.T, on0)
        back = Tensor.empty([300, 200], "float", device="cuda:1")
        ops.copy(on0.T, back)
        torch.cuda.synchronize(0); torch.cuda.synchronize(1)
        assert np.array_equal(on0.numpy(), m.T.astype(np.float64))
        assert np.array_equal(back.numpy(), m)
