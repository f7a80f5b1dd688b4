"""Host logic of the multi-GPU path, run as two gloo ranks on CPU: the leading-axis shards tile
the tensor exactly, and per-rank partial results combined by the collective equal the result over
the whole tensor (the per-rank partials are computed by the numpy oracle here; on GPUs they come
from solid_gpu_axpy_sums_float)."""
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest

from solid_b200 import shard

ROOT = Path(__file__).resolve().parent.parent


def test_shard_ranges_tile_the_axis():
    for n in (0, 1, 7, 8, 1000, 2 ** 32, 2 ** 32 + 5):
        for world in (1, 2, 3, 4, 8):
            bounds = [shard.shard_range(n, r, world) for r in range(world)]
            assert bounds[0][0] == 0 and bounds[-1][1] == n
            for (lo, hi), (lo2, _) in zip(bounds, bounds[1:]):
                assert lo <= hi == lo2
            sizes = [hi - lo for lo, hi in bounds]
            assert max(sizes) == (n + world - 1) // world
    with pytest.raises(ValueError):
        shard.shard_range(10, 2, 2)
    with pytest.raises(KeyError):
        shard.combine(None, "median")


def test_peer_exchange_is_not_offered_without_a_process_group():
    # the peer-memory exchange needs an initialised NCCL group of at least two ranks; otherwise callers use combine()
    assert shard.PeerSum.create("cpu") is None


def _worker(rank, world, port, n, q):
    sys.path[:0] = [str(ROOT), str(ROOT / "ocean-tensor-package_b200")]
    import torch
    import torch.distributed as dist
    from oracle import solid_numpy as sn
    from solid_b200 import shard as sh
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rng = np.random.default_rng(42)                       # every rank draws the same full tensors
        x = rng.uniform(-1, 1, n).astype(np.float32)
        y = rng.uniform(-1, 1, n).astype(np.float32)
        lo, hi = sh.shard_range(n, rank, world)
        z = sn.axpy("float", 0.5, x[lo:hi], y[lo:hi])         # the shard's elementwise result
        part = torch.tensor([z.astype(np.float64).sum(), (z.astype(np.float64) ** 2).sum()], dtype=torch.float64)
        sh.combine(part, "sum")
        mx = torch.tensor([z.max() if z.size else -np.inf], dtype=torch.float64)
        sh.combine(mx, "maximum")
        nz = torch.tensor([int((z != 0).sum())], dtype=torch.int64)
        sh.combine(nz, "nnz")
        anyv = torch.tensor([int((z > 0.99).any())], dtype=torch.int64)
        sh.combine(anyv, "any")
        allv = torch.tensor([int((z > -2).all())], dtype=torch.int64)
        sh.combine(allv, "all")
        full = sn.axpy("float", 0.5, x, y).astype(np.float64)
        ok = (abs(part[0].item() - full.sum()) <= 1e-9 * np.abs(full).sum()
              and abs(sh.finish_norm2(part[1]) - np.sqrt((full ** 2).sum())) <= 1e-9 * np.sqrt((full ** 2).sum())
              and mx.item() == full.max() and nz.item() == int((full != 0).sum())
              and anyv.item() == int((full > 0.99).any()) and allv.item() == int((full > -2).all()))
        q.put((rank, bool(ok), (lo, hi)))
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(120)
def test_two_rank_combination_matches_whole_tensor():
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    world, n = 2, 100003
    procs = [ctx.Process(target=_worker, args=(r, world, port, n, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=100) for _ in range(world)]
    for p in procs:
        p.join(timeout=30)
        assert p.exitcode == 0
    assert all(ok for _, ok, _ in results), results
    ranges = sorted(r for _, _, r in results)
    assert ranges[0][0] == 0 and ranges[0][1] == ranges[1][0] and ranges[1][1] == n
