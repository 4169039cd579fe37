"""Sequence sharding with gathered K/V on the GPU: the block plan with the library's kernels on one GPU (every
rank's calls made in turn on the whole K and V, no collective involved) and, where two GPUs are visible, two NCCL
ranks against the oracle on the whole sequence."""
import math
import os
import socket

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

import oracle

pytestmark = pytest.mark.gpu


def _problem(B, H, S, D, seed):
    g = torch.Generator().manual_seed(seed)
    return tuple((torch.randn((B, H, S, D), generator=g) * 0.5).bfloat16() for _ in range(4))


def _reference(q, k, v, do, scale, causal):
    f = lambda t: t.float().numpy()
    o, lse = oracle.attn_fwd(f(q), f(k), f(v), scale, causal, None, None, 0.0)
    return (o, lse) + tuple(oracle.attn_bwd(f(q), f(k), f(v), f(do), scale, causal, None, None, 0.0))


def _errors(got, ref, idx):
    out = []
    for g, r in zip(got, ref):
        r = r[:, :, idx]
        out.append(float(np.abs(g.float().cpu().numpy() - r).max() / (2e-3 + np.abs(r).max() * 2 ** -8)))
    return out


@pytest.mark.parametrize("causal", [False, True])
def test_block_plan_with_the_kernels_on_one_gpu(ctx, causal):
    """world = 1 equals the direct call; and the calls of every rank of a world of four, made one after the other on
    one GPU against the whole K and V, give every rank's rows of O, lse and dQ, and dK / dV shares that sum to the
    whole gradients."""
    from cuda_ltc_b200 import gather, ring
    B, H, S, D = 1, 2, 1536, 64
    scale = 1 / math.sqrt(D)
    q, k, v, do = _problem(B, H, S, D, 31)
    ref = _reference(q, k, v, do, scale, causal)
    dq_, dk_, dv_ = ref[2], ref[3], ref[4]
    tq, tk, tv, tdo = (t.cuda() for t in (q, k, v, do))
    ops = ring.CudaOps(ctx, scale, comm_sms=0)
    o, lse, kf, vf = gather.gathered_attention_fwd(ops, tq, tk, tv, 0, 1, causal)
    grads = gather.gathered_attention_bwd(ops, tq, kf, vf, o, lse, tdo, 0, 1, causal)
    assert max(_errors((o, lse) + tuple(grads), ref, np.arange(S))) < 1.5
    world = 4
    dk_sum = np.zeros_like(dk_, dtype=np.float64)
    dv_sum = np.zeros_like(dv_, dtype=np.float64)
    for rank in range(world):
        idx = ring.owned_positions(S, world, rank, causal)
        ql, dol = (t.index_select(2, idx.cuda()).contiguous() for t in (tq, tdo))
        L = ql.shape[2]
        o_r = torch.empty_like(ql)
        lse_r = torch.empty((B, H, L), dtype=torch.float32, device="cuda")
        dq_r = torch.empty_like(ql)
        for r0, n, nk in gather._query_blocks(rank, world, L, causal):
            lb = torch.empty((B, H, n), dtype=torch.float32, device="cuda")
            ops.block_fwd(ql[:, :, r0:r0 + n], tk[:, :, :nk], tv[:, :, :nk], causal, out=o_r[:, :, r0:r0 + n], lse=lb)
            lse_r[:, :, r0:r0 + n] = lb
            dk_p = torch.empty((B, H, nk, D), dtype=torch.bfloat16, device="cuda")
            dv_p = torch.empty_like(dk_p)
            ops.block_bwd(ql[:, :, r0:r0 + n], tk[:, :, :nk], tv[:, :, :nk], o_r[:, :, r0:r0 + n], lb,
                          dol[:, :, r0:r0 + n], causal, dq=dq_r[:, :, r0:r0 + n], dk=dk_p, dv=dv_p)
            dk_sum[:, :, :nk] += dk_p.float().cpu().numpy()
            dv_sum[:, :, :nk] += dv_p.float().cpu().numpy()
        assert max(_errors((o_r, lse_r, dq_r), (ref[0], ref[1], dq_), idx.numpy())) < 1.5, rank
    torch.cuda.synchronize()
    assert ctx.device_status() == 0
    # eight partial results, each rounded to bf16, were added: a few units of rounding
    for s_, r_ in ((dk_sum, dk_), (dv_sum, dv_)):
        assert np.abs(s_ - r_).max() < 4 * (2e-3 + np.abs(r_).max() * 2 ** -8)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _nccl_worker(rank, world, port, out):
    import torch.distributed as dist
    from cuda_ltc_b200 import Context, gather, ring
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        ctx = Context(rank)
        B, H, S, D = 1, 4, 2048, 64
        scale = 1 / math.sqrt(D)
        q, k, v, do = _problem(B, H, S, D, 21)                 # the same whole problem on every rank
        ref = _reference(q, k, v, do, scale, True)
        mine = [ring.shard_sequence(x.cuda(), world, rank, True) for x in (q, k, v, do)]
        ops, cache = ring.CudaOps(ctx, scale, comm_sms=0), {}
        worst = 0.0
        for _ in range(2):                                     # the second pass runs on reused buffers
            o, lse, kf, vf = gather.gathered_attention_fwd(ops, *mine[:3], rank, world, True, cache=cache)
            grads = gather.gathered_attention_bwd(ops, mine[0], kf, vf, o, lse, mine[3], rank, world, True,
                                                  cache=cache)
            torch.cuda.synchronize()
            idx = ring.owned_positions(S, world, rank, True).numpy()
            worst = max(worst, max(_errors((o, lse) + tuple(grads), ref, idx)))
        # the shares of dK / dV summed in bf16: one more rounding of each rank's share
        g16 = gather.gathered_attention_bwd(ops, mine[0], kf, vf, o, lse, mine[3], rank, world, True, cache=cache,
                                            reduce_in_bf16=True)
        torch.cuda.synchronize()
        worst16 = max(_errors(tuple(g16), ref[2:], idx))
        out[rank] = (max(worst, worst16 / 2), ctx.device_status())
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_nccl_ranks_equal_the_whole_sequence():
    world = 2
    out = mp.Manager().dict()
    mp.spawn(_nccl_worker, args=(world, _free_port(), out), nprocs=world, join=True)
    for r in range(world):
        worst, status = out[r]
        assert worst < 1.5 and status == 0, f"rank {r}: {worst}"
