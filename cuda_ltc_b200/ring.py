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

    def __init__(self, ctx, scale=None, mode=None, comm_sms=16):
        """``comm_sms``: SMs left free while slices are in flight.  The attention kernels are persistent (one
        CTA per SM for the whole launch), so without free SMs the communication library's copy kernels would
        only start when an attention kernel ends and the exchange would not overlap the arithmetic."""
        from . import _lib
        self.ctx, self.scale, self.comm_sms = ctx, scale, comm_sms
        self.mode = _lib.MODE_AUTO if mode is None else mode

    def begin(self):
        # The exchange (torch.distributed P2P) orders itself against torch's CURRENT stream at call time; the
        # context's kernels must run on that same stream, or they would race with the K/V receives.
        import torch
        self.ctx.set_stream(torch.cuda.current_stream(self.ctx.device))
        if self.comm_sms > 0:
            self.ctx.set_sm_limit(max(1, self.ctx.sm_count() - self.comm_sms))

    def end(self):
        self.ctx.set_sm_limit(0)

    def block_fwd(self, q, k, v, causal, out=None, lse=None):
        return self.ctx.attn_fwd(q, k, v, scale=self.scale, causal=causal, mode=self.mode, out=out, lse=lse)

    def merge(self, o_acc, lse_acc, o_blk, lse_blk, s0):
        self.ctx.attn_merge(o_acc, lse_acc, o_blk, lse_blk, s0)

    def block_bwd(self, q, k, v, o, lse, dout, causal, dq=None, dk=None, dv=None):
        return self.ctx.attn_bwd(q, k, v, o, lse, dout, scale=self.scale, causal=causal, mode=self.mode,
                                 dq=dq, dk=dk, dv=dv)

    def accumulate(self, acc, part, s0):
        self.ctx.accumulate_rows(acc, part, s0)


# ---- buffers -----------------------------------------------------------------------------------------------
def _buf(cache, name, shape, dtype, device):
    """A scratch tensor that lives in ``cache`` across calls (steady-state steps then allocate nothing; the
    allocator would otherwise stall the host on every hop, because tensors handed to the communication stream
    are not reusable at once).  With ``cache`` None a fresh tensor is returned."""
    if cache is None:
        return torch.empty(shape, dtype=dtype, device=device)
    key = (name, tuple(shape), dtype, str(device))
    t = cache.get(key)
    if t is None:
        t = cache[key] = torch.empty(shape, dtype=dtype, device=device)
    return t


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

    def __init__(self, rank: int, world: int, group=None, cache=None):
        self.rank, self.world, self.group, self.cache = rank, world, group, cache
        self._hop = {}

    def start(self, tensors: List[torch.Tensor], tag: str = "x") -> _Transfer:
        """``tag`` names the stream of messages (K/V, gradients): its hops alternate between two sets of
        receive buffers, so a hop never lands in the buffers the next hop is being sent from."""
        import torch.distributed as dist
        hop = self._hop[tag] = self._hop.get(tag, -1) + 1
        received = [_buf(self.cache, f"recv.{tag}.{hop & 1}.{i}", t.shape, t.dtype, t.device)
                    for i, t in enumerate(tensors)]
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
    def __init__(self, ops, q, k, v, rank, world, causal, cache=None):
        self.ops, self.q, self.rank, self.world, self.causal, self.cache = ops, q, rank, world, causal, cache
        self.kv = [k, v]                                       # the slice currently held (two messages per hop)
        B, H, L, D = q.shape
        self.o_acc = _buf(cache, "o_acc", (B, H, L, D), torch.float32, q.device)
        self.lse_acc = _buf(cache, "lse_acc", (B, H, L), torch.float32, q.device)

    def compute(self, step):
        q = self.q
        B, H, L, D = q.shape
        src = (self.rank - step) % self.world
        (qs, qn), (ks, kn), cz = block_plan(self.rank, src, L, self.causal)
        o_blk = _buf(self.cache, "o_blk", (B, H, qn, D), q.dtype, q.device)
        if step == 0:
            # the rank's own slice covers every local row: its result starts the accumulators
            self.ops.block_fwd(q, self.kv[0], self.kv[1], cz, out=o_blk, lse=self.lse_acc)
            self.o_acc.copy_(o_blk)
            return
        lse_blk = _buf(self.cache, "lse_blk", (B, H, qn), torch.float32, q.device)
        self.ops.block_fwd(q[:, :, qs:qs + qn], self.kv[0][:, :, ks:ks + kn], self.kv[1][:, :, ks:ks + kn], cz,
                           out=o_blk, lse=lse_blk)
        self.ops.merge(self.o_acc, self.lse_acc, o_blk, lse_blk, qs)

    def result(self):
        return self.o_acc.to(self.q.dtype, copy=True), self.lse_acc.clone()


class _Backward:
    def __init__(self, ops, q, k, v, o, lse, dout, rank, world, causal, cache=None):
        self.ops, self.q, self.o, self.lse, self.dout = ops, q, o, lse, dout
        self.rank, self.world, self.causal, self.cache = rank, world, causal, cache
        self.kv = [k, v]
        f32 = torch.float32
        # fp32 [dK, dV] of the slice currently held; they travel with it
        self.dkv = [_buf(cache, "dk_acc", k.shape, f32, q.device), _buf(cache, "dv_acc", v.shape, f32, q.device)]
        self.dq_acc = _buf(cache, "dq_acc", q.shape, f32, q.device)
        c = q.shape[2] // 2
        self._lse_hi = lse[:, :, c:].contiguous() if causal and world > 1 else None

    def kernels(self, step):
        """The step's partial gradients (dq, dk, dv) and the rows they belong to."""
        q = self.q
        B, H, L, D = q.shape
        src = (self.rank - step) % self.world
        (qs, qn), (ks, kn), cz = block_plan(self.rank, src, L, self.causal)
        lse = self.lse if qn == L else self._lse_hi
        rows = slice(qs, qs + qn)
        outs = dict(dq=_buf(self.cache, "dq_blk", (B, H, qn, D), q.dtype, q.device),
                    dk=_buf(self.cache, "dk_blk", (B, H, kn, D), q.dtype, q.device),
                    dv=_buf(self.cache, "dv_blk", (B, H, kn, D), q.dtype, q.device))
        parts = self.ops.block_bwd(q[:, :, rows], self.kv[0][:, :, ks:ks + kn], self.kv[1][:, :, ks:ks + kn],
                                   self.o[:, :, rows], lse, self.dout[:, :, rows], cz, **outs)
        return parts, qs, ks

    def absorb(self, step, parts, qs, ks):
        dq, dk, dv = parts
        if step == 0:                                          # own slice: full rows on both sides
            self.dq_acc.copy_(dq)
            self.dkv[0].copy_(dk)
            self.dkv[1].copy_(dv)
            return
        self.ops.accumulate(self.dq_acc, dq, qs)
        self.ops.accumulate(self.dkv[0], dk, ks)
        self.ops.accumulate(self.dkv[1], dv, ks)

    def result(self):
        dt = self.q.dtype
        return tuple(t.to(dt, copy=True) for t in (self.dq_acc, self.dkv[0], self.dkv[1]))


# ---- drivers -----------------------------------------------------------------------------------------------
def ring_attention_fwd(ops, q, k, v, rank, world, causal=False, exchange=None, cache=None):
    """Forward of the rank's query slice against the whole sequence.  q, k, v: the rank's slices
    [B, H, L, D] (``shard_sequence``), contiguous.  Returns (o [B, H, L, D] in q's dtype, lse [B, H, L] fp32).
    ``cache``: a dict the caller keeps between calls; all scratch and receive buffers then live in it."""
    if world == 1:
        return ops.block_fwd(q, k, v, causal)
    exchange = exchange or RingExchange(rank, world, cache=cache)
    st = _Forward(ops, q, k, v, rank, world, causal, cache)
    getattr(ops, "begin", lambda: None)()
    try:
        for step in range(world):
            moving = exchange.start(st.kv, "kv") if step + 1 < world else None   # arrives during this step
            st.compute(step)
            if moving is not None:
                st.kv = moving.wait()
    finally:
        getattr(ops, "end", lambda: None)()
    return st.result()


def ring_attention_bwd(ops, q, k, v, o, lse, dout, rank, world, causal=False, exchange=None, cache=None):
    """Backward of ``ring_attention_fwd``: (dq, dk, dv) of the rank's slices."""
    if world == 1:
        return ops.block_bwd(q, k, v, o, lse, dout, causal)
    exchange = exchange or RingExchange(rank, world, cache=cache)
    st = _Backward(ops, q, k, v, o, lse, dout, rank, world, causal, cache)
    arriving = None
    dt = q.dtype
    getattr(ops, "begin", lambda: None)()
    try:
        for step in range(world):
            last = step + 1 == world
            moving = exchange.start(st.kv, "kv") if not last else None
            parts = st.kernels(step)                 # runs while the previous hop of the gradients is in flight
            if arriving is not None:
                st.dkv = arriving.wait()
            st.absorb(step, *parts)
            # the gradient accumulators follow their slice once this rank has added its share; after the last
            # step they belong to rank+1, so the same hop brings every slice's gradients home.  Nothing is added
            # after that hop, so it carries the gradients already rounded to the output type (half the bytes).
            if last and dt != torch.float32:
                home = [_buf(cache, f"home.{i}", t.shape, dt, t.device) for i, t in enumerate(st.dkv)]
                for h, t in zip(home, st.dkv):
                    h.copy_(t)
                arriving = exchange.start(home, "home")
            else:
                arriving = exchange.start(st.dkv, "dkv")
            if moving is not None:
                st.kv = moving.wait()
    finally:
        getattr(ops, "end", lambda: None)()
    dq = st.dq_acc.to(dt, copy=True)             # while the hop home is in flight
    dk, dv = arriving.wait()
    return dq, dk.to(dt, copy=True), dv.to(dt, copy=True)


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
            s.absorb(step, *s.kernels(step))
        if step + 1 < world:
            _rotate(states, "kv")
        if world > 1:
            _rotate(states, "dkv")
    return [s.result() for s in states]
