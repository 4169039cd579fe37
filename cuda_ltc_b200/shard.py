"""Partition of the attention work over the GPUs of one box.

The attention core is independent per (batch, head) pair, so the pairs are dealt out to the
ranks in contiguous, balanced ranges and no rank ever needs another rank's data: there is no
collective on the data path.  The only communication of a multi-GPU run is the reduction of
the per-rank timings (maximum over ranks) and, for checks, of a few scalars.

The whole module (projections around the core) shards by sequences with replicated weights:
forward and the input gradient stay local, and only the weight gradients, which are sums over
rows, need one sum over the ranks (``sum_weight_grads``).

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


class _Pending:
    """Handle of a weight-gradient sum in flight: ``wait()`` finishes it and scatters the bucket back."""

    def __init__(self, work, bucket, grads, all_grads=None):
        self._work, self._bucket, self._grads = work, bucket, grads
        self._all = grads if all_grads is None else all_grads

    def wait(self):
        if self._work is not None:
            self._work.wait()
            self._work = None
        off = 0
        for g in self._grads:                      # empty when the sum ran in place on the gradients' own memory
            n = g.numel()
            g.copy_(self._bucket[off:off + n].view_as(g))
            off += n
        return self._all


def _as_one_allocation(grads):
    """One flat tensor aliasing all of ``grads`` if they are back-to-back contiguous views of one
    allocation (as ``Context.tsa_bwd`` returns them), else None."""
    first = grads[0]
    off = first.storage_offset()
    for g in grads:
        if (not g.is_contiguous() or g.dtype != first.dtype or g.device != first.device
                or g.untyped_storage().data_ptr() != first.untyped_storage().data_ptr()
                or g.storage_offset() != off):
            return None
        off += g.numel()
    return first.as_strided((off - first.storage_offset(),), (1,), first.storage_offset())


def sum_weight_grads(grads, group=None, async_op=False):
    """Sum each rank's partial weight gradients over the ranks, in place, with ONE collective.

    With sequences dealt out over the ranks and the weights replicated, dWq, dWk, dWv, dWo (and the
    bias / LayerNorm gradients) of a rank cover only its rows; the full gradient is their sum.  The
    tensors are packed into one bucket (4 MiB for four 512 x 512 fp32 matrices) so the cost is one
    launch, not one per matrix.  ``async_op=True`` returns a handle whose ``wait()`` completes the sum,
    so the caller can run the previous layer's backward meanwhile.  Without a process group the
    gradients are returned unchanged.
    """
    import torch
    import torch.distributed as dist
    grads = [g for g in grads if g is not None]
    if not grads or not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return _Pending(None, None, [], grads) if async_op else grads   # wait() hands the gradients back
    packed = _as_one_allocation(grads)
    bucket = packed if packed is not None else torch.cat([g.reshape(-1) for g in grads])
    work = dist.all_reduce(bucket, op=dist.ReduceOp.SUM, group=group, async_op=True)
    pending = _Pending(work, bucket, [] if packed is not None else grads, grads)
    return pending if async_op else pending.wait()
