"""Known answers taken from the golden outputs of the reference's own GPU example scripts
(examples/python/gpu/tensors/*.ref, printed to five digits).  Each case states the file it was
read from.  The inputs are rebuilt here and pushed (1) through the numpy restatement of the
oracle on CPU and (2) through the CUDA library behind the Ocean-style host API on the GPU; both
must print the reference's numbers."""
import numpy as np
import pytest

from oracle import solid_numpy as sn


def close5(got, want):
    got, want = np.asarray(got, dtype=np.float64).reshape(-1), np.asarray(want, dtype=np.float64).reshape(-1)
    return got.shape == want.shape and np.all(np.abs(got - want) <= 6e-6 * np.maximum(1.0, np.abs(want)))


def half_values(bits):
    return np.asarray(bits, dtype=np.uint16).view(np.float16).astype(np.float64)


# ----------------------------------------------------------------------------- CPU: numpy oracle
def test_axis_reduce_04_oracle():
    """ocean_axis_reduce_04.ref: A = arange(24) as float 2x3x4 (column-major)."""
    A = np.arange(24, dtype=np.float32).reshape((2, 3, 4), order="F")
    assert close5(sn.reduce_axis("norm2", "float", A, (0, 1)), [7.41620, 21.23676, 35.76311, 50.38849])
    F = A[:, ::-1, :]                                           # A.fliplr(True)
    assert np.array_equal(sn.reduce_axis("minimum", "float", F, 0), np.array([[4, 10, 16, 22], [2, 8, 14, 20], [0, 6, 12, 18]]))
    assert np.array_equal(sn.reduce_axis("maximum", "float", F, 2), np.array([[22, 20, 18], [23, 21, 19]]))
    n3 = sn.reduce_axis("norm", "float", F, (0, 1), p=3.0)
    assert close5(n3, [6.08220, 16.04544, 26.70881, 37.50774])
    assert close5(half_values(sn.convert("float", "half", n3)), [6.08203, 16.04688, 26.70313, 37.50000])


def test_small_reductions_oracle():
    """ocean_sumabs_01.ref, ocean_sum_02.ref, ocean_all_01.ref, ocean_maximumabs_01.ref."""
    assert sn.reduce_all("sum_abs", "int64", np.array([1, -2, 3])) == 6
    for dtype in ("int8", "int16", "half", "chalf", "cdouble"):
        x = sn.convert("double", dtype, np.array([1.0, -2.0, 5.0]))
        v = sn.reduce_all("sum_abs", dtype, x)
        v = half_values([v])[0] if dtype in ("half", "chalf") else float(v)
        assert v == 8
        y = sn.convert("double", dtype, np.array([1.0, 2.0, 5.0]))
        s = sn.reduce_all("sum", dtype, y)
        if dtype == "half":
            s = half_values([s])[0]
        elif dtype == "chalf":
            s = half_values([s["real"]])[0]
        assert complex(s) == 8
    assert sn.reduce_all("sum", "bool", np.array([1, 0, 1], dtype=np.uint8)) == 2
    assert sn.reduce_all("all", "int64", np.array([1, 1, 1, 1, 0, 1])) == 0
    A = np.array([1 + 2j, 3 + 1j, 1, 2 + 2j])
    assert close5(sn.reduce_all("maximum_abs", "cdouble", A), 3.16228)


BITSHIFT = {   # ocean_bitshift_01.ref: a = [0,1,2,9], b = [0,1,2,4,6,8]; rows are shift counts
    "int8": [[0, 1, 2, 9], [0, 2, 4, 18], [0, 4, 8, 36], [0, 16, 32, -112], [0, 64, -128, 64], [0, 0, 0, 0]],
    "uint8": [[0, 1, 2, 9], [0, 2, 4, 18], [0, 4, 8, 36], [0, 16, 32, 144], [0, 64, 128, 64], [0, 0, 0, 0]],
    "uint32": [[0, 1, 2, 9], [0, 2, 4, 18], [0, 4, 8, 36], [0, 16, 32, 144], [0, 64, 128, 576], [0, 256, 512, 2304]],
    "bool": [[0, 1, 1, 1]] + [[0, 0, 0, 0]] * 5,
}


def test_elementwise_known_answers_oracle():
    for dtype, table in BITSHIFT.items():
        a = sn.convert("int64", dtype, np.array([0, 1, 2, 9]))
        for shift, row in zip([0, 1, 2, 4, 6, 8], table):
            got = sn.binary("bitshift_left", dtype, a, np.full(4, shift, dtype=np.int8))
            assert np.array_equal(got.astype(np.int64), np.array(row)), (dtype, shift)
    # ocean_power_01.ref
    assert np.array_equal(sn.binary("power", "int8", np.array([1, 2, 3, 4], dtype=np.int8), np.full(4, 2, dtype=np.int16)), [1, 4, 9, 16])
    r = sn.binary("power", "float", np.array([1, 2, 3, 4], dtype=np.float32), np.full(4, 0.5, dtype=np.float32))
    assert close5(r, [1.0, 1.41421, 1.73205, 2.0])
    h = sn.binary("power", "half", sn.float_to_half(np.array([1, 2, 3, 4], dtype=np.float32)), sn.float_to_half(np.full(4, 0.5, dtype=np.float32)))
    assert close5(half_values(h), [1.0, 1.41406, 1.73242, 2.0])
    # ocean_min_01.ref (int8 block; the NaN entry was cast to 0)
    v1, v2 = np.array([1, 2, 3, 1, 0, 2, 4], dtype=np.int8), np.array([3, 2, 1, 1, 1, 2, 4], dtype=np.int8)
    assert np.array_equal(sn.binary("min", "int8", v1, v2), [1, 2, 1, 1, 0, 2, 4])
    assert np.array_equal(sn.binary("max", "int8", v1, v2), [3, 2, 3, 1, 1, 2, 4])
    # ocean_fabs_01.ref
    z = np.array([-3 - 4j])
    assert sn.unary("fabs", "cdouble", z)[0] == 5 and sn.unary("absolute", "cdouble", z)[0] == 5
    assert sn.unary("fabs", "int8", np.array([-3], dtype=np.int8))[0] == 3
    # ocean_unary_01.ref: square of int8 [1,2,3] delivered as int16
    assert np.array_equal(sn.convert("int8", "int16", sn.unary("square", "int8", np.array([1, 2, 3], dtype=np.int8))), [1, 4, 9])


# ----------------------------------------------------------------------------- GPU: the product
@pytest.mark.gpu
def test_axis_reduce_04_gpu(gpu):
    from solid_b200 import Tensor, ops
    A = Tensor.from_numpy(np.arange(24, dtype=np.float32).reshape((2, 3, 4), order="F"))
    assert close5(ops.reduce_axis("norm2", A, [0, 1]).numpy(), [7.41620, 21.23676, 35.76311, 50.38849])
    F = A.slice(1, 2, -1, -1)                                   # fliplr: negative stride along axis 1
    assert F.size == [2, 3, 4]
    assert np.array_equal(ops.minimum(F, 0).numpy(), np.array([[4, 10, 16, 22], [2, 8, 14, 20], [0, 6, 12, 18]]))
    assert np.array_equal(ops.maximum(F, 2, keepdims=True).numpy()[:, :, 0], np.array([[22, 20, 18], [23, 21, 19]]))
    n3 = ops.norm(F, 3, [0, 1])
    assert close5(n3.numpy(), [6.08220, 16.04544, 26.70881, 37.50774])
    B = Tensor.empty([4], "half")
    ops.copy(n3, B)
    assert close5(half_values(B.numpy()), [6.08203, 16.04688, 26.70313, 37.50000])


@pytest.mark.gpu
def test_small_reductions_gpu(gpu):
    from solid_b200 import Tensor, ops
    assert ops.sum_abs(Tensor.from_numpy(np.array([1, -2, 3], dtype=np.int64))) == 6
    base = Tensor.from_numpy(np.array([1.0, -2.0, 5.0]))
    pos = Tensor.from_numpy(np.array([1.0, 2.0, 5.0]))
    for dtype in ("int8", "int16", "half", "chalf", "cdouble"):
        v = ops.sum_abs(ops.cast(base, dtype))
        assert (half_values([v])[0] if dtype in ("half", "chalf") else float(v)) == 8
        s = ops.sum(ops.cast(pos, dtype))
        if dtype == "half":
            s = half_values([s])[0]
        elif dtype == "chalf":
            s = half_values([s["real"]])[0]
        assert complex(s) == 8
    assert ops.sum(Tensor.from_numpy(np.array([1, 0, 1], dtype=np.uint8), "bool")) == 2
    assert ops.all(Tensor.from_numpy(np.array([1, 1, 1, 1, 0, 1], dtype=np.int64))) == 0
    assert close5(ops.maximum_abs(Tensor.from_numpy(np.array([1 + 2j, 3 + 1j, 1, 2 + 2j]))), 3.16228)
    with pytest.raises(Exception, match="empty"):
        ops.maximum_abs(Tensor.empty([0], "double"))            # "does not apply to empty tensors"


@pytest.mark.gpu
def test_elementwise_known_answers_gpu(gpu):
    from solid_b200 import Tensor, ops
    shifts = Tensor.from_numpy(np.array([0, 1, 2, 4, 6, 8], dtype=np.uint8))
    for dtype, table in BITSHIFT.items():
        a = ops.cast(Tensor.from_numpy(np.array([0, 1, 2, 9], dtype=np.int64)), dtype)
        # a is 1x4 ('r' row vector), the shift counts 6(x1): broadcast to 6x4
        a_row = a.as_strided([1, 4], [0, a.elemsize])
        s_col = shifts.as_strided([6, 1], [1, 0])
        got = ops.binary("bitshift_left", a_row, s_col).numpy().astype(np.int64)
        assert np.array_equal(got, np.array(table)), dtype
    x = Tensor.from_numpy(np.array([1, 2, 3, 4], dtype=np.int8))
    two = Tensor.from_numpy(np.array([2], dtype=np.int16)).as_strided([4], [0])
    assert np.array_equal(ops.binary("power", x, two).numpy(), [1, 4, 9, 16])
    xf = Tensor.from_numpy(np.array([1, 2, 3, 4], dtype=np.float32))
    hf = Tensor.from_numpy(np.array([0.5], dtype=np.float32)).as_strided([4], [0])
    assert close5(ops.binary("power", xf, hf).numpy(), [1.0, 1.41421, 1.73205, 2.0])
    assert close5(half_values(ops.binary("power", ops.cast(xf, "half"), ops.cast(hf, "half")).numpy()), [1.0, 1.41406, 1.73242, 2.0])
    v1 = Tensor.from_numpy(np.array([1, 2, 3, 1, 0, 2, 4], dtype=np.int8)); v2 = Tensor.from_numpy(np.array([3, 2, 1, 1, 1, 2, 4], dtype=np.int8))
    assert np.array_equal(ops.binary("min", v1, v2).numpy(), [1, 2, 1, 1, 0, 2, 4])
    assert np.array_equal(ops.binary("max", v1, v2).numpy(), [3, 2, 3, 1, 1, 2, 4])
    r2 = Tensor.empty([7], "cfloat")
    ops.binary("fmin", v1, v2, r2)                               # result delivered in another dtype
    assert np.array_equal(r2.numpy(), np.array([1, 2, 1, 1, 0, 2, 4], dtype=np.complex64))
    z = Tensor.from_numpy(np.array([-3 - 4j]))
    assert ops.fabs(z).numpy()[0] == 5 and ops.absolute(z).numpy()[0] == 5
    # ocean_sign_01.ref, complex-half block
    vals = np.array([-1, 0, 1, 1 + 2j, 0 + 2j, 0 - 2j, 0 + 0j])
    sg = ops.sign(ops.cast(Tensor.from_numpy(vals), "chalf"))
    b = Tensor.empty([7], "int8"); ops.copy(sg, b)
    assert np.array_equal(b.numpy(), [-1, 0, 1, 1, 1, -1, 0])
    # ocean_unary_01.ref: square of int8 into an int16 result, also with a byte-swapped destination
    q = Tensor.empty([3], "int16")
    ops.unary("square", Tensor.from_numpy(np.array([1, 2, 3], dtype=np.int8)), q)
    assert np.array_equal(q.numpy(), [1, 4, 9])
    qs = Tensor.empty([3], "int16"); qs.byteswapped = True
    ops.unary("square", Tensor.from_numpy(np.array([1, 2, 3], dtype=np.int8)), qs)
    assert np.array_equal(qs.numpy(), [1, 4, 9])
    assert np.array_equal(qs.storage[:6].cpu().numpy().view(">i2"), [1, 4, 9])   # stored big-endian
    # tensor_add_01.ref: C is a 5x3 view with strides (3,1) elements over the first 15 of 100 floats
    store = Tensor.from_numpy(np.concatenate([np.arange(15), np.zeros(85)]).astype(np.float32))
    C = store.as_strided([5, 3], [12, 4])
    hundred = Tensor.from_numpy(np.array([100], dtype=np.float32)).as_strided([5, 3], [0, 0])
    ops.add(C, hundred, C)
    assert np.array_equal(store.numpy(), np.concatenate([np.arange(15) + 100, np.zeros(85)]).astype(np.float32))
