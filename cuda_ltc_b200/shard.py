"""Partition of the attention work over the GPUs of one box.

The attention core is independent per (batch, head) pair, so the pairs are dealt out to the
ranks in contiguous, balanced ranges and no rank ever needs another rank's data: there is no
collective on the data path.  The only communication of a multi-GPU run is the reduction of
the per-rank timings (maximum over ranks) and, for checks, of a few scalars.

The reference is single-GPU (its only device selection is ``cudaSetDevice(0)`` in a test,
src/ml/time_self_attention_test.cu:523); this module has no counterpart there.
"""
from __future__ import annotations

from typing import List, Tuple


def unit_range(n_units: int, world: int, rank: int) -> range:
    """Contiguous range of units (batch x head pairs, or sequences) owned by ``rank``.

    The first ``n_units % world`` ranks get one unit more; every unit has exactly one owner.
    """
    if world < 1 or not (0 <= rank < world):
        raise ValueError(f"bad rank {rank} of {world}")
    if n_units < 0:
        raise ValueError("n_units must be non-negative")
    base, extra = divmod(n_units, world)
    start = rank * base + min(rank, extra)
    return range(start, start + base + (1 if rank < extra else 0))


def batch_slices(batch: int, heads: int, world: int, rank: int) -> List[Tuple[int, int, int]]:
    """The rank's units as (batch index, first head, one-past-last head) runs.

    Sharding by whole sequences keeps per-sequence key lengths local; when ``batch`` is not a
    multiple of ``world`` the split falls inside a sequence's heads.
    """
    r = unit_range(batch * heads, world, rank)
    out: List[Tuple[int, int, int]] = []
    u = r.start
    while u < r.stop:
        b, h0 = divmod(u, heads)
        h1 = min(heads, h0 + (r.stop - u))
        out.append((b, h0, h1))
        u += h1 - h0
    return out


def reduce_max(values, group=None):
    """Element-wise maximum over the ranks of a list of floats (identity without a process group)."""
    import torch
    import torch.distributed as dist
    t = torch.tensor(list(values), dtype=torch.float64)
    if dist.is_available() and dist.is_initialized():
        backend = dist.get_backend(group)
        if backend == "nccl":
            t = t.cuda()
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return t.cpu().tolist()
