"""Sequence sharding of one long attention problem with GATHERED keys and values.

The second way (beside ``cuda_ltc_b200.ring``) to deal one sequence out over the GPUs of a box.  Every rank keeps a
slice of the positions of Q, K and V (the same layout as the ring: ``ring.shard_sequence``, zig-zag under a causal
mask).  Forward: one all-gather brings every rank the whole K and V; the rank then attends its own queries to them
with the ordinary forward kernel, so there is nothing to merge.  Backward: the ordinary backward kernel gives dQ for
the rank's queries and the rank's share of dK / dV for ALL keys; one reduce-scatter (fp32) sums the shares and
leaves every rank the gradients of the keys it owns.

Against the ring this trades memory (the whole K and V, and an fp32 dK / dV of the whole sequence, live on every
rank: 1.6 GB at B=8 H=16 S=16384 D=64) for two collectives that run at NVLink / NVSwitch bandwidth instead of
2 * world point-to-point hops, and for kernels that see long key ranges instead of slice pairs.

Causal masking.  A kernel call hides key j from query i when j > i + (Sk - Sq), so a block of queries that starts at
global position p attends, causally, to the PREFIX of the keys that ends with the block: Sq = block length,
Sk = p + block length.  With the zig-zag layout a rank owns chunks r and 2 * world - 1 - r of 2 * world chunks of
length c: two calls, keys [0, (r + 1) c) and [0, (2 * world - r) c), the same total work on every rank.

The arithmetic goes through an ``ops`` object as in ``ring`` (``ring.CudaOps`` for the library's kernels); the
collectives are ``torch.distributed`` (NCCL between GPUs, gloo in the CPU tests).  The reference is single-GPU and
has no counterpart of this module.
"""
from __future__ import annotations

from typing import List, Tuple

import torch

from .ring import _buf


def _dist():
    import torch.distributed as dist
    return dist


def _query_blocks(rank: int, world: int, local_len: int, causal: bool) -> List[Tuple[int, int, int]]:
    """(first local row, rows, keys visible) of the calls a rank makes; keys visible = length of the key prefix."""
    if not causal:
        return [(0, local_len, world * local_len)]
    c = local_len // 2
    return [(0, c, (rank + 1) * c), (c, c, (2 * world - rank) * c)]


def gather_sequence(x: torch.Tensor, world: int, causal: bool, group=None, cache=None, name="g") -> torch.Tensor:
    """All ranks' slices of a [B, H, L, D] tensor, put back into sequence order: [B, H, world * L, D]."""
    if world == 1:
        return x
    dist = _dist()
    flat = _buf(cache, name + "_all", (world,) + tuple(x.shape), x.dtype, x.device)
    dist.all_gather_into_tensor(flat.view(-1), x.contiguous().view(-1), group=group)
    B, H, L, D = x.shape
    full = _buf(cache, name + "_full", (B, H, world * L, D), x.dtype, x.device)
    if not causal:
        # rank r holds positions [r L, (r + 1) L): [world, B, H, L, D] -> [B, H, world, L, D]
        full.view(B, H, world, L, D).copy_(flat.permute(1, 2, 0, 3, 4))
        return full
    # zig-zag: the first halves of the slices are chunks 0 .. world - 1 in rank order, the second halves are
    # chunks 2 world - 1 .. world, i.e. the rest of the sequence in REVERSE rank order
    c = L // 2
    both = full.view(B, H, 2, world, c, D)
    both[:, :, 0].copy_(flat[:, :, :, :c].permute(1, 2, 0, 3, 4))
    both[:, :, 1].copy_(flat[:, :, :, c:].permute(1, 2, 0, 3, 4).flip(2))
    return full


def gathered_attention_fwd(ops, q, k, v, rank, world, causal=False, group=None, cache=None):
    """Forward for this rank's queries.  q, k, v: the rank's slices [B, H, L, D] (``ring.shard_sequence``).
    Returns (o, lse, k_full, v_full); the gathered K and V are handed back for the backward pass."""
    B, H, L, D = q.shape
    if causal and L % 2:
        raise ValueError("the zig-zag layout needs an even slice length")
    if hasattr(ops, "begin"):
        ops.begin()
    try:
        k_full = gather_sequence(k, world, causal, group, cache, "k")
        v_full = gather_sequence(v, world, causal, group, cache, "v")
        o = torch.empty_like(q)
        lse = torch.empty((B, H, L), dtype=torch.float32, device=q.device)
        for r0, n, nk in _query_blocks(rank, world, L, causal):
            lse_blk = _buf(cache, f"lse_blk{r0}", (B, H, n), torch.float32, q.device)      # the kernels want it dense
            ops.block_fwd(q[:, :, r0:r0 + n], k_full[:, :, :nk], v_full[:, :, :nk], causal,
                          out=o[:, :, r0:r0 + n], lse=lse_blk)
            lse[:, :, r0:r0 + n].copy_(lse_blk)
    finally:
        if hasattr(ops, "end"):
            ops.end()
    return o, lse, k_full, v_full


def _add_shares(send: torch.Tensor, t: int, part: torch.Tensor, world: int, L: int, causal: bool) -> None:
    """send[owner, t] += the owner's rows of ``part`` (gradients of the first part.shape[2] keys, sequence order)."""
    B, H, nk, D = part.shape
    if not causal:
        send[:, t].add_(part.view(B, H, world, L, D).permute(2, 0, 1, 3, 4))
        return
    c = L // 2
    m = nk // c                                             # chunks of the key prefix; chunk j belongs to rank j or,
    m1 = min(m, world)                                      # in the second half, to rank 2 world - 1 - j
    send[:m1, t, :, :, :c].add_(part[:, :, :m1 * c].view(B, H, m1, c, D).permute(2, 0, 1, 3, 4))
    if m > world:
        tail = part[:, :, world * c:m * c].view(B, H, m - world, c, D).permute(2, 0, 1, 3, 4).flip(0)
        send[2 * world - m:world, t, :, :, c:].add_(tail)


def gathered_attention_bwd(ops, q, k_full, v_full, o, lse, dout, rank, world, causal=False, group=None, cache=None,
                           reduce_in_bf16=False):
    """Backward for this rank's queries: (dq, dk, dv) for the rank's slices.  k_full, v_full: what the forward
    returned.  ``reduce_in_bf16``: the shares of dK / dV travel and are summed as bf16 (half the bytes of the
    reduce-scatter; one more rounding per hop) instead of fp32."""
    B, H, L, D = q.shape
    if hasattr(ops, "begin"):
        ops.begin()
    try:
        dq = torch.empty_like(q)
        # this rank's shares of the gradients of every key, fp32, grouped by the rank that owns the key
        send = _buf(cache, "dkv_send", (world, 2, B, H, L, D), torch.float32, q.device)
        send.zero_()
        for r0, n, nk in _query_blocks(rank, world, L, causal):
            dk_p = _buf(cache, f"dk_part{r0}", (B, H, nk, D), q.dtype, q.device)
            dv_p = _buf(cache, f"dv_part{r0}", (B, H, nk, D), q.dtype, q.device)
            ops.block_bwd(q[:, :, r0:r0 + n], k_full[:, :, :nk], v_full[:, :, :nk], o[:, :, r0:r0 + n],
                          lse[:, :, r0:r0 + n].contiguous(), dout[:, :, r0:r0 + n], causal, dq=dq[:, :, r0:r0 + n],
                          dk=dk_p, dv=dv_p)
            _add_shares(send, 0, dk_p, world, L, causal)
            _add_shares(send, 1, dv_p, world, L, causal)
        if world == 1:
            return dq, send[0, 0].to(q.dtype), send[0, 1].to(q.dtype)
        dist = _dist()
        if reduce_in_bf16 and q.dtype == torch.bfloat16:
            send_x = _buf(cache, "dkv_send16", tuple(send.shape), torch.bfloat16, q.device)
            send_x.copy_(send)
        else:
            send_x = send
        recv = _buf(cache, "dkv_recv", (2, B, H, L, D), send_x.dtype, q.device)
        if dist.get_backend(group) == "gloo":
            # (no reduce-scatter in that backend: sum everywhere and keep the own part)
            dist.all_reduce(send_x, group=group)
            recv.copy_(send_x[rank])
        else:
            dist.reduce_scatter_tensor(recv.view(-1), send_x.view(-1), group=group)
    finally:
        if hasattr(ops, "end"):
            ops.end()
    return dq, recv[0].to(q.dtype), recv[1].to(q.dtype)
