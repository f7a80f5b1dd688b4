"""Leading-axis sharding of large tensors over the GPUs of one node.

Ocean itself has no collectives (tensors are split by hand with tensor.split(axis, devices),
docs/python/module_core.md:1155-1164 of the reference); this module adds the one exchange the
sharded reductions need.  Rank g of G owns the contiguous element range
[g*ceil(n/G), min(n, (g+1)*ceil(n/G))) of the outermost axis in its own HBM; elementwise work
needs no communication, a reduction combines one small tensor of per-GPU partial results with
a collective of the matching kind.  The process group is whatever torch.distributed was
initialised with (NCCL over NVLink on GPUs, gloo in the CPU tests of the host logic).

For the pair {sum, sum of squares} there is a second route on GPUs: PeerSum exchanges the pairs through peer
memory with one small kernel of this library (solid_gpu_peer_sum_float), which takes a few microseconds where an
all-reduce call of two floats takes 10-17; it needs exchange buffers every GPU can address, which torch's symmetric
memory provides.  When that cannot be set up the NCCL route is used.
"""
from __future__ import annotations

import math
import os
import sys

COMBINE = {"sum": "SUM", "sum_abs": "SUM", "nnz": "SUM", "sumsq": "SUM",
           "maximum": "MAX", "maximum_abs": "MAX", "any": "MAX",
           "minimum": "MIN", "minimum_abs": "MIN", "all": "MIN"}


def shard_range(n: int, rank: int, world: int) -> tuple[int, int]:
    """Element range [lo, hi) of the leading axis owned by `rank` ("as evenly as possible":
    equal ceil(n/world) chunks, the last ranks may own fewer or none)."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError("rank %d of %d" % (rank, world))
    per = (n + world - 1) // world
    lo = min(rank * per, n)
    return lo, min(lo + per, n)


def combine(partials, kind: str, group=None):
    """All-reduce a tensor of per-rank partial results in place with the collective that matches
    the reduction (`kind` is a reduction name, or "sumsq" for the squared sum behind norm2)."""
    import torch.distributed as dist
    if kind not in COMBINE:
        raise KeyError("no collective defined for reduction %r" % kind)
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(partials, op=getattr(dist.ReduceOp, COMBINE[kind]), group=group)
    return partials


class PeerSum:
    """Exchange of a pair of floats per GPU through peer memory (one kernel per exchange, bounded wait).

    `PeerSum.create(device)` returns None when the process group is not NCCL, has one rank, or symmetric memory
    cannot be set up; callers then use `combine`.  All ranks must call `sum_pair` the same number of times."""

    def __init__(self, lib, world, rank, buffers, symm, handle, device):
        import torch
        self.lib, self.world, self.rank, self.buffers = lib, world, rank, buffers
        self._keep = (symm, handle)                      # the mapping lives as long as these
        self.sequence = 0
        self.status = torch.zeros(1, dtype=torch.int32, device=device)

    @staticmethod
    def create(device, group=None):
        import torch
        import torch.distributed as dist
        if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) < 2:
            return None
        if dist.get_backend(group) != "nccl" or os.environ.get("SOLID_B200_EXCHANGE", "peer") != "peer":
            return None
        from . import _lib
        lib = _lib.get()
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        ok, made = 1, None
        # the exchange uses plain peer stores only: keep the buffers off NVLink multicast objects
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        try:
            import torch.distributed._symmetric_memory as symm_mem
            nbytes = lib.peer_sum_buffer_size(world)
            symm = symm_mem.empty(max(nbytes // 4, 4), dtype=torch.float32, device=device)
            symm.zero_()
            handle = symm_mem.rendezvous(symm, group if group is not None else dist.group.WORLD)
            made = PeerSum(lib, world, rank, [int(p) for p in handle.buffer_ptrs], symm, handle, device)
            torch.cuda.synchronize(device)
        except Exception as exc:                         # no symmetric memory on this machine: every rank must agree
            ok = 0
            print("[shard] peer exchange unavailable (%s: %s); using the NCCL all-reduce" % (type(exc).__name__, exc),
                  file=sys.stderr, flush=True)
        flag = torch.tensor([ok], dtype=torch.int32, device=device)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=group)     # also orders the zeroing before the first exchange
        return made if int(flag.item()) == 1 else None

    def sum_pair(self, pair, sqrt_second=False, stream=None):
        """pair: float32 CUDA tensor of two elements, replaced by the sums over all ranks (the second one by the
        square root of its sum when sqrt_second)."""
        import torch
        self.sequence += 1
        if self.sequence >= 1 << 32:
            raise OverflowError("PeerSum sequence exhausted")
        s = torch.cuda.current_stream().cuda_stream if stream is None else stream
        self.lib.peer_sum_float(self.world, self.rank, self.buffers, self.sequence, 2, pair.data_ptr(), pair.data_ptr(),
                                2 if sqrt_second else 0, 0, self.status.data_ptr(), s)
        return pair

    def check(self):
        """Raise if some exchange gave up waiting for a peer (reads one int from the device)."""
        if int(self.status.item()) != 0:
            raise RuntimeError("a peer did not deliver its partial sums within the limit")


def finish_norm2(sumsq):
    """norm2 from the combined sum of squares (the square root is taken after the exchange)."""
    return math.sqrt(float(sumsq))


def sharded_axpy_sums(a, x, y, z=None, sums=None, group=None, peer=None):
    """z = a*x + y on this rank's shard with sum(z) and sum(z*z) combined over all ranks.
    Returns (z, sums) with sums = {sum(z), sum(z*z)} of the WHOLE tensor on every rank (device); with a PeerSum
    the pairs are exchanged through peer memory, else by the collective."""
    from . import ops
    z, sums = ops.axpy_sums(a, x, y, z, sums)
    if peer is not None:
        peer.sum_pair(sums)
    else:
        combine(sums, "sum", group)
    return z, sums
