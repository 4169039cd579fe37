"""Sequence sharding of one long attention problem over the GPUs of a box, with a ring exchange of K/V.

The headline partition of this library is by (batch, head) and needs no communication
(``cuda_ltc_b200.shard``).  This module is the optional second partition for sequences too long for that to
be enough: every rank keeps a slice of the positions of Q, K and V; the K/V slices travel round the ring
(rank r sends to r+1, receives from r-1) and at each of the ``world`` steps a rank attends its own queries
to the slice it currently holds, folding the partial result into running (O, log-sum-exp) accumulators
(``ltca_attn_merge``).  The backward makes the same tour with the dK/dV accumulators travelling beside their
K/V slice, plus one last hop that brings them home; dQ accumulates locally.  The partial backward of a
(query slice, key slice) pair is the ordinary backward kernel run with the FINAL log-sum-exp and output of
the query rows, which makes the pair's contribution exact without any correction afterwards.

Causal masking uses the zig-zag layout: the sequence is cut into 2*world chunks and rank r owns chunks r and
2*world-1-r, so that every rank has the same amount of unmasked work at every step:
  * the slice of the rank itself: ordinary causal attention over its two chunks (the second chunk lies
    entirely after the first, so the concatenation's causal mask is the true one);
  * a slice from a lower rank: all local queries see that slice's FIRST chunk and nothing of its second;
  * a slice from a higher rank: only the local SECOND chunk sees anything, and it sees the whole slice.

The exchange runs through ``torch.distributed`` point-to-point operations (NCCL over NVLink between GPUs,
gloo in the CPU tests); the arithmetic of every step goes through an ``ops`` object, ``CudaOps`` for the
library's kernels.  ``ring_attention_*_emulated`` runs all ranks of the same schedule inside one process (one
GPU), moving the slices by reference, for checking the schedule without several devices.

The reference is single-GPU and has no counterpart of this module.
"""
from __future__ import annotations

from typing import List, Sequence, Tuple

import torch


# ---- layout ------------------------------------------------------------------------------------------------
def owned_positions(seq_len: int, world: int, rank: int, causal: bool) -> torch.Tensor:
    """Global positions held by ``rank``, in local order."""
    if world < 1 or not (0 <= rank < world):
        raise ValueError(f"bad rank {rank} of {world}")
    parts = 2 * world if causal else world
    if seq_len % parts:
        raise ValueError(f"sequence length {seq_len} is not a multiple of {parts}")
    c = seq_len // parts
    if not causal:
        return torch.arange(rank * c, (rank + 1) * c)
    hi = 2 * world - 1 - rank
    return torch.cat([torch.arange(rank * c, (rank + 1) * c), torch.arange(hi * c, (hi + 1) * c)])


def shard_sequence(x: torch.Tensor, world: int, rank: int, causal: bool) -> torch.Tensor:
    """The rank's slice of a [B, H, S, D] (or [B, H, S]) tensor, contiguous."""
    idx = owned_positions(x.shape[2], world, rank, causal).to(x.device)
    return x.index_select(2, idx).contiguous()


def unshard_sequence(parts: Sequence[torch.Tensor], causal: bool) -> torch.Tensor:
    """Inverse of ``shard_sequence`` over all ranks' slices (given in rank order)."""
    world = len(parts)
    seq_len = sum(p.shape[2] for p in parts)
    shape = list(parts[0].shape)
    shape[2] = seq_len
    out = torch.empty(shape, dtype=parts[0].dtype, device=parts[0].device)
    for r, p in enumerate(parts):
        out.index_copy_(2, owned_positions(seq_len, world, r, causal).to(p.device), p)
    return out


def block_plan(rank: int, src: int, local_len: int, causal: bool) -> Tuple[Tuple[int, int], Tuple[int, int], bool]:
    """What ``rank`` computes against the slice that started at ``src``:
    ((first query row, rows), (first key row, rows), causal mask inside the pair)."""
    if not causal:
        return (0, local_len), (0, local_len), False
    c = local_len // 2
    if src == rank:
        return (0, local_len), (0, local_len), True
    if src < rank:
        return (0, local_len), (0, c), False
    return (c, c), (0, local_len), False


# ---- arithmetic of one step --------------------------------------------------------------------------------
class CudaOps:
    """The steps' arithmetic on this library's kernels (``Context``); raises if the library is missing."""

    def __init__(self, ctx, scale=None, mode=None):
        from . import _lib
        self.ctx, self.scale = ctx, scale
        self.mode = _lib.MODE_AUTO if mode is None else mode

    def block_fwd(self, q, k, v, causal):
        return self.ctx.attn_fwd(q, k, v, scale=self.scale, causal=causal, mode=self.mode)

    def merge(self, o_acc, lse_acc, o_blk, lse_blk, s0):
        self.ctx.attn_merge(o_acc, lse_acc, o_blk, lse_blk, s0)

    def block_bwd(self, q, k, v, o, lse, dout, causal):
        return self.ctx.attn_bwd(q, k, v, o, lse, dout, scale=self.scale, causal=causal, mode=self.mode)

    def accumulate(self, acc, part, s0):
        self.ctx.accumulate_rows(acc, part, s0)


# ---- exchange ----------------------------------------------------------------------------------------------
class _Transfer:
    def __init__(self, reqs, received):
        self._reqs, self._received = reqs, received

    def wait(self):
        for r in self._reqs:
            r.wait()
        self._reqs = []
        return self._received


class RingExchange:
    """Sends tensors to rank+1 and receives the same shapes from rank-1 (one batched P2P call per hop)."""

    def __init__(self, rank: int, world: int, group=None):
        self.rank, self.world, self.group = rank, world, group

    def start(self, tensors: List[torch.Tensor]) -> _Transfer:
        import torch.distributed as dist
        received = [torch.empty_like(t) for t in tensors]
        nxt, prv = (self.rank + 1) % self.world, (self.rank - 1) % self.world
        if self.group is not None:
            nxt, prv = dist.get_global_rank(self.group, nxt), dist.get_global_rank(self.group, prv)
        ops = []
        for t, r in zip(tensors, received):
            ops.append(dist.P2POp(dist.isend, t, nxt, self.group))
            ops.append(dist.P2POp(dist.irecv, r, prv, self.group))
        return _Transfer(dist.batch_isend_irecv(ops), received)


# ---- per-rank state ----------------------------------------------------------------------------------------
class _Forward:
    def __init__(self, ops, q, k, v, rank, world, causal):
        self.ops, self.q, self.rank, self.world, self.causal = ops, q, rank, world, causal
        B, H, L, D = q.shape
        self.kv = torch.stack([k, v]).contiguous()             # [2, B, H, L, D]: one message per hop
        self.o_acc = torch.zeros((B, H, L, D), dtype=torch.float32, device=q.device)
        self.lse_acc = torch.full((B, H, L), float("-inf"), dtype=torch.float32, device=q.device)

    def compute(self, step):
        src = (self.rank - step) % self.world
        (qs, qn), (ks, kn), cz = block_plan(self.rank, src, self.q.shape[2], self.causal)
        o_blk, lse_blk = self.ops.block_fwd(self.q[:, :, qs:qs + qn], self.kv[0][:, :, ks:ks + kn],
                                            self.kv[1][:, :, ks:ks + kn], cz)
        self.ops.merge(self.o_acc, self.lse_acc, o_blk, lse_blk, qs)

    def result(self):
        return self.o_acc.to(self.q.dtype), self.lse_acc


class _Backward:
    def __init__(self, ops, q, k, v, o, lse, dout, rank, world, causal):
        self.ops, self.q, self.o, self.lse, self.dout = ops, q, o, lse, dout
        self.rank, self.world, self.causal = rank, world, causal
        self.kv = torch.stack([k, v]).contiguous()
        self.dkv = torch.zeros(self.kv.shape, dtype=torch.float32, device=q.device)   # travels with kv
        self.dq_acc = torch.zeros(q.shape, dtype=torch.float32, device=q.device)
        c = q.shape[2] // 2
        self._lse_hi = lse[:, :, c:].contiguous() if causal else None

    def compute(self, step):
        src = (self.rank - step) % self.world
        L = self.q.shape[2]
        (qs, qn), (ks, kn), cz = block_plan(self.rank, src, L, self.causal)
        lse = self.lse if qn == L else self._lse_hi
        rows = slice(qs, qs + qn)
        dq, dk, dv = self.ops.block_bwd(self.q[:, :, rows], self.kv[0][:, :, ks:ks + kn],
                                        self.kv[1][:, :, ks:ks + kn], self.o[:, :, rows], lse,
                                        self.dout[:, :, rows], cz)
        self.ops.accumulate(self.dq_acc, dq, qs)
        self.ops.accumulate(self.dkv[0], dk, ks)
        self.ops.accumulate(self.dkv[1], dv, ks)

    def result(self):
        dt = self.q.dtype
        return self.dq_acc.to(dt), self.dkv[0].to(dt), self.dkv[1].to(dt)


# ---- drivers -----------------------------------------------------------------------------------------------
def ring_attention_fwd(ops, q, k, v, rank, world, causal=False, exchange=None):
    """Forward of the rank's query slice against the whole sequence.  q, k, v: the rank's slices
    [B, H, L, D] (``shard_sequence``).  Returns (o [B, H, L, D] in q's dtype, lse [B, H, L] fp32)."""
    exchange = exchange or RingExchange(rank, world)
    st = _Forward(ops, q, k, v, rank, world, causal)
    for step in range(world):
        moving = exchange.start([st.kv]) if step + 1 < world else None   # next slice arrives during this step
        st.compute(step)
        if moving is not None:
            st.kv = moving.wait()[0]
    return st.result()


def ring_attention_bwd(ops, q, k, v, o, lse, dout, rank, world, causal=False, exchange=None):
    """Backward of ``ring_attention_fwd``: (dq, dk, dv) of the rank's slices."""
    exchange = exchange or RingExchange(rank, world)
    st = _Backward(ops, q, k, v, o, lse, dout, rank, world, causal)
    for step in range(world):
        moving = exchange.start([st.kv]) if step + 1 < world else None
        st.compute(step)
        # the gradient accumulators follow their slice once this rank has added its share; after the last
        # step they belong to rank+1, so the same hop brings every slice's gradients home
        grads = exchange.start([st.dkv]) if world > 1 else None
        if moving is not None:
            st.kv = moving.wait()[0]
        if grads is not None:
            st.dkv = grads.wait()[0]
    return st.result()


def _rotate(states, name):
    held = [getattr(s, name) for s in states]
    for r, s in enumerate(states):
        setattr(s, name, held[(r - 1) % len(states)])


def ring_attention_fwd_emulated(ops, qs, ks, vs, causal=False):
    """All ranks of the forward schedule in one process: lists of per-rank slices in, list of (o, lse) out."""
    world = len(qs)
    states = [_Forward(ops, qs[r], ks[r], vs[r], r, world, causal) for r in range(world)]
    for step in range(world):
        for s in states:
            s.compute(step)
        if step + 1 < world:
            _rotate(states, "kv")
    return [s.result() for s in states]


def ring_attention_bwd_emulated(ops, qs, ks, vs, os_, lses, douts, causal=False):
    """All ranks of the backward schedule in one process; returns a list of (dq, dk, dv) per rank."""
    world = len(qs)
    states = [_Backward(ops, qs[r], ks[r], vs[r], os_[r], lses[r], douts[r], r, world, causal)
              for r in range(world)]
    for step in range(world):
        for s in states:
            s.compute(step)
        if step + 1 < world:
            _rotate(states, "kv")
        if world > 1:
            _rotate(states, "dkv")
    return [s.result() for s in states]
