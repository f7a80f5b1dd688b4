"""Leading-axis sharding of large tensors over the GPUs of one node.

Ocean itself has no collectives (tensors are split by hand with tensor.split(axis, devices),
docs/python/module_core.md:1155-1164 of the reference); this module adds the one exchange the
sharded reductions need.  Rank g of G owns the contiguous element range
[g*ceil(n/G), min(n, (g+1)*ceil(n/G))) of the outermost axis in its own HBM; elementwise work
needs no communication, a reduction combines one small tensor of per-GPU partial results with
a collective of the matching kind.  The process group is whatever torch.distributed was
initialised with (NCCL over NVLink on GPUs, gloo in the CPU tests of the host logic).
"""
from __future__ import annotations

import math

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


def finish_norm2(sumsq):
    """norm2 from the combined sum of squares (the square root is taken after the exchange)."""
    return math.sqrt(float(sumsq))


def sharded_axpy_sums(a, x, y, z=None, sums=None, group=None):
    """z = a*x + y on this rank's shard with sum(z) and sum(z*z) combined over all ranks.
    Returns (z, sums) with sums = {sum(z), sum(z*z)} of the WHOLE tensor on every rank (device)."""
    from . import ops
    z, sums = ops.axpy_sums(a, x, y, z, sums)
    combine(sums, "sum", group)
    return z, sums
