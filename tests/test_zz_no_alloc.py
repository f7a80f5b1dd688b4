"""solid_gpu_axis_sum_float_noalloc against solid_gpu_axis_sum_float, through the C-ABI.

The no-alloc variant exists for callers that cannot request device memory where they reduce
(allocator lock held, no tolerance for the device-wide synchronisation of cudaMalloc/cudaFree,
memory budget already handed out): its scratch is an array inside the library image.  Both entry
points run the same kernels with the same plan, so their results must be identical bit for bit
(the tolerance of the axis-sum parity tests, 1e-5*sqrt(n), is not even needed).  Two calls are made
in a row because the array keeps the previous call's contents.  This file sorts last so that a run
stopping at the first failure has already executed every other test.
"""
import ctypes as C

import numpy as np
import pytest

import util
from solid_b200 import dtypes as dt

pytestmark = pytest.mark.gpu

CASES = [((4096, 64), (0,)),       # dense axis: one warp or block per output, no scratch needed
         ((64, 4096), (1,)),       # strided axis, few outputs: the reduced range is split over blocks -> scratch
         ((8192, 8), (0,)),        # few outputs, long dense rows: split over blocks -> scratch
         ((5, 6, 7), (0, 2)),
         ((1 << 20,), (0,))]       # ONE output split over a wave of blocks: the last block to arrive folds the partials


def run_pair(gpu, dev, shape, axes, seed):
    rng = np.random.default_rng(seed)
    v = util.dense_view("float", list(shape), pad_elems=4)
    buf = util.fill_buffer(v, rng)
    keep = [i for i in range(len(shape)) if i not in axes]
    size = [shape[i] for i in keep]; st1 = [v.strides[i] for i in keep]
    rsize = [shape[i] for i in axes]; rst = [v.strides[i] for i in axes]
    vo = util.dense_view("float", size)
    d = dev.upload(buf)
    outs = []
    for variant in ("regular", "noalloc"):
        do = dev.upload(np.zeros(vo.nbytes, dtype=np.uint8))
        cfg = gpu.reduce_axis_prepare(dt.WORKSIZE["float"], size, st1, d.data_ptr(), vo.strides, do.data_ptr(), rsize, rst, dev.stream)
        if variant == "regular":
            scratch = dev.empty(cfg.bufferSize + 16)
            cfg.data.ptrBuffer = scratch.data_ptr() if cfg.bufferSize else None
            gpu.reduce_axis("axis_sum", "float", cfg)
        else:
            assert cfg.bufferSize <= gpu.noalloc_scratch_size()
            gpu.axis_sum_float_noalloc(cfg)
            assert cfg.data.ptrBuffer is None              # the caller's structure is not modified
        outs.append(util.gather(dev.download(do), vo))
    # and both agree with a float64 sum within the axis-sum tolerance of the parity tests
    arr = util.gather(buf, v).reshape(shape, order="F").astype(np.float64)
    want = arr.sum(axis=tuple(axes)).reshape(-1, order="F")
    n = int(np.prod(rsize))
    bound = util.accumulation_bound(n, "float", np.abs(arr).sum(axis=tuple(axes)).reshape(-1, order="F"))
    assert np.all(np.abs(outs[1].astype(np.float64) - want) <= bound)
    return cfg.bufferSize, outs


def test_noalloc_axis_sum_matches_regular_entry_point_twice(gpu):
    dev = util.Device()
    used_scratch = False
    for shape, axes in CASES:
        for call in range(2):                                   # two calls in a row on the shared array
            size, (regular, noalloc) = run_pair(gpu, dev, shape, axes, seed=17 + call)
            used_scratch |= size > 0
            assert np.array_equal(regular.view(np.uint32), noalloc.view(np.uint32)), (shape, axes, call)
    assert used_scratch, "no case exercised the built-in scratch array"


def test_noalloc_rejects_plans_beyond_its_scratch(gpu):
    from solid_b200._lib import SolidError
    dev = util.Device()
    limit = gpu.noalloc_scratch_size()
    assert limit == 1 << 20
    d = dev.empty(1 << 12); do = dev.empty(1 << 12)
    cfg = gpu.reduce_axis_prepare(4, [8], [4], d.data_ptr(), [4], do.data_ptr(), [16], [32], dev.stream)
    cfg.bufferSize = limit + 1                                  # a plan that asks for more than the array holds
    with pytest.raises(SolidError, match="scratch"):
        gpu.axis_sum_float_noalloc(cfg)
