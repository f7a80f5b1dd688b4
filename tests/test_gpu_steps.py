"""Parity of the range kernels solid_gpu_steps_{int64,double,cdouble}_<type> with the reference's
Solid CPU library (solid/src/core/cpu/template_steps.c): element i, counted in the column-major
order of the tensor's own dimensions, is offset + i * step cast to the element type.

Bit-exact on every type.  The cases include the reference's corners: negative int64 offsets into
floating-point tensors (the position is unsigned there, so the sum wraps before the cast), values
outside the range of the integer element types, and steps that do not round exactly in double.
"""
import numpy as np
import pytest

import util
from solid_b200 import dtypes as dt
from solid_b200 import oplist as ol

pytestmark = pytest.mark.gpu


def views(dtype):
    es = dt.SIZE[dtype]
    out = [("contig%d" % n, util.dense_view(dtype, [n])) for n in (0, 1, 7, 1000, 4099)]
    out.append(("offset", util.dense_view(dtype, [1003], offset_elems=3)))
    out.append(("matrix", util.dense_view(dtype, [32, 9])))
    out.append(("padded", util.dense_view(dtype, [13, 7], pad_elems=3)))
    v = util.dense_view(dtype, [11, 37])
    out.append(("transposed", util.View(dtype, [37, 11], [v.strides[1], v.strides[0]], 0, v.nbytes)))
    v3 = util.dense_view(dtype, [5, 6, 7])
    out.append(("reversed_dim", util.View(dtype, [5, 6, 7], [v3.strides[0], -v3.strides[1], v3.strides[2]],
                                          5 * v3.strides[1], v3.nbytes)))
    out.append(("unit_dims", util.View(dtype, [1, 40, 1, 3], [es, es, 40 * es, 40 * es], 0, 120 * es + 64)))
    out.append(("zero_dim", util.dense_view(dtype, [])))
    return out


CASES = {
    "int64": [(0, 1), (-5, 3), (7, -2), (2 ** 40, 2 ** 33), (-1, 0)],
    "double": [(0.0, 1.0), (-2.5, 0.1), (1e6, -3.75), (0.3, 1e-3), (-1e10, 7e7)],
    "cdouble": [(1 - 2j, 0.5 + 0.25j), (-3.5 + 0j, 0.1 - 1e-3j)],
}


@pytest.mark.parametrize("kind", ["int64", "double", "cdouble"])
def test_steps_match_reference(kind, gpu, cpu):
    dev = util.Device()
    for dtype in dt.GROUPS[ol.STEPS_OPS["steps_" + kind]]:
        rng = np.random.default_rng(31 + dt.INDEX[dtype])
        for name, v in views(dtype):
            for offset, step in CASES[kind]:
                base = util.fill_buffer(v, rng, "general")
                want = base.copy()
                cpu.steps(kind, dtype, v.size, v.strides, want.ctypes.data + v.offset, offset, step)
                d = dev.upload(base)
                gpu.steps(kind, dtype, v.size, v.strides, d.data_ptr() + v.offset, offset, step, dev.stream)
                got = dev.download(d)
                # the whole buffer: elements outside the view must be untouched
                assert np.array_equal(got, want), ("steps_%s_%s" % (kind, dtype), name, offset, step,
                                                   np.nonzero(got != want)[0][:4])


def test_steps_errors(gpu):
    from solid_b200._lib import SolidError
    dev = util.Device()
    d = dev.empty(256)
    with pytest.raises(SolidError, match="dimensions"):
        gpu.steps("double", "float", [2] * 9, [4] * 9, d.data_ptr(), 0.0, 1.0, dev.stream)
    with pytest.raises(SolidError, match="aligned"):
        gpu.steps("int64", "int32", [8], [4], d.data_ptr() + 2, 0, 1, dev.stream)
