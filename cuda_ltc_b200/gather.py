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

from .ring import _buf, owned_positions, unshard_sequence


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
    if not causal:
        # rank r holds positions [r L, (r + 1) L): [world, B, H, L, D] -> [B, H, world, L, D]
        full = _buf(cache, name + "_full", (x.shape[0], x.shape[1], world * x.shape[2], x.shape[3]), x.dtype, x.device)
        full.view(x.shape[0], x.shape[1], world, x.shape[2], x.shape[3]).copy_(flat.permute(1, 2, 0, 3, 4))
        return full
    return unshard_sequence(list(flat.unbind(0)), causal)


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


def gathered_attention_bwd(ops, q, k_full, v_full, o, lse, dout, rank, world, causal=False, group=None, cache=None):
    """Backward for this rank's queries: (dq, dk, dv) for the rank's slices.  k_full, v_full: what the forward
    returned."""
    B, H, L, D = q.shape
    S = k_full.shape[2]
    if hasattr(ops, "begin"):
        ops.begin()
    try:
        dq = torch.empty_like(q)
        # this rank's share of the gradients of every key, fp32, in sequence order
        dk_acc = _buf(cache, "dk_acc", (B, H, S, D), torch.float32, q.device)
        dv_acc = _buf(cache, "dv_acc", (B, H, S, D), torch.float32, q.device)
        dk_acc.zero_()
        dv_acc.zero_()
        for r0, n, nk in _query_blocks(rank, world, L, causal):
            dk_p = _buf(cache, f"dk_part{r0}", (B, H, nk, D), q.dtype, q.device)
            dv_p = _buf(cache, f"dv_part{r0}", (B, H, nk, D), q.dtype, q.device)
            ops.block_bwd(q[:, :, r0:r0 + n], k_full[:, :, :nk], v_full[:, :, :nk], o[:, :, r0:r0 + n],
                          lse[:, :, r0:r0 + n].contiguous(), dout[:, :, r0:r0 + n], causal, dq=dq[:, :, r0:r0 + n],
                          dk=dk_p, dv=dv_p)
            ops.accumulate(dk_acc, dk_p, 0)
            ops.accumulate(dv_acc, dv_p, 0)
        if world == 1:
            return dq, dk_acc.to(q.dtype), dv_acc.to(q.dtype)
        # owner-major order, then one reduce-scatter for both gradients
        dist = _dist()
        send = _buf(cache, "dkv_send", (world, 2, B, H, L, D), torch.float32, q.device)
        for r in range(world):
            idx = owned_positions(S, world, r, causal).to(q.device)
            torch.index_select(dk_acc, 2, idx, out=send[r, 0])
            torch.index_select(dv_acc, 2, idx, out=send[r, 1])
        recv = _buf(cache, "dkv_recv", (2, B, H, L, D), torch.float32, q.device)
        if dist.get_backend(group) == "gloo":
            # (no reduce-scatter in that backend: sum everywhere and keep the own part)
            dist.all_reduce(send, group=group)
            recv.copy_(send[rank])
        else:
            dist.reduce_scatter_tensor(recv.view(-1), send.view(-1), group=group)
    finally:
        if hasattr(ops, "end"):
            ops.end()
    return dq, recv[0].to(q.dtype), recv[1].to(q.dtype)
