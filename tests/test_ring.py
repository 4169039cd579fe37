"""Sequence sharding with a ring exchange of K/V (cuda_ltc_b200/ring.py).

CPU: the schedule (zig-zag causal layout, which pairs are computed, the travelling dK/dV accumulators, the
home hop) is checked with fp64 numpy arithmetic standing in for the kernels, once with all ranks emulated in
one process and once as two gloo ranks that really exchange their slices.  GPU: the same schedule on the
library's kernels, all ranks emulated on the one device, against the oracle on the whole sequence.
"""
import math
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from cuda_ltc_b200 import ring


class NumpyOps:
    """fp64 stand-in for the kernels: one (query slice, key slice) pair at a time."""

    def __init__(self, scale):
        self.scale = scale

    def _scores(self, q, k, causal):
        s = np.einsum("bhid,bhjd->bhij", q.numpy().astype(np.float64), k.numpy().astype(np.float64)) * self.scale
        if causal:
            i, j = np.arange(s.shape[2])[:, None], np.arange(s.shape[3])[None, :]
            s = np.where(j <= i, s, -np.inf)
        return s

    def block_fwd(self, q, k, v, causal, out=None, lse=None):
        s = self._scores(q, k, causal)
        m = s.max(-1, keepdims=True)
        p = np.exp(s - m)
        l = p.sum(-1, keepdims=True)
        o = np.einsum("bhij,bhjd->bhid", p / l, v.numpy().astype(np.float64))
        o, l = torch.from_numpy(o), torch.from_numpy((m + np.log(l))[..., 0]).float()
        if out is not None:
            out.copy_(o)
            lse.copy_(l)
            return out, lse
        return o, l

    def merge(self, o_acc, lse_acc, o_blk, lse_blk, s0):
        n = o_blk.shape[2]
        la, lb = lse_acc[:, :, s0:s0 + n].double(), lse_blk.double()
        new = torch.logaddexp(la, lb)
        o_acc[:, :, s0:s0 + n] = (o_acc[:, :, s0:s0 + n].double() * torch.exp(la - new)[..., None]
                                  + o_blk.double() * torch.exp(lb - new)[..., None]).float()
        lse_acc[:, :, s0:s0 + n] = new.float()

    def block_bwd(self, q, k, v, o, lse, dout, causal, dq=None, dk=None, dv=None):
        outs = (dq, dk, dv)
        s = self._scores(q, k, causal)
        p = np.exp(s - lse.numpy().astype(np.float64)[..., None])
        do = dout.numpy().astype(np.float64)
        dv = np.einsum("bhij,bhid->bhjd", p, do)
        dp = np.einsum("bhid,bhjd->bhij", do, v.numpy().astype(np.float64))
        delta = (do * o.numpy().astype(np.float64)).sum(-1, keepdims=True)
        ds = p * (dp - delta) * self.scale
        dq = np.einsum("bhij,bhjd->bhid", ds, k.numpy().astype(np.float64))
        dk = np.einsum("bhij,bhid->bhjd", ds, q.numpy().astype(np.float64))
        for dst, a in zip(outs, (dq, dk, dv)):
            dst.copy_(torch.from_numpy(a))
        return outs

    def accumulate(self, acc, part, s0):
        acc[:, :, s0:s0 + part.shape[2]] += part.float()


def _problem(B, H, S, D, seed):
    g = torch.Generator().manual_seed(seed)
    return tuple(torch.randn((B, H, S, D), generator=g) * 0.5 for _ in range(4))


def _oracle(q, k, v, do, scale, causal):
    o, lse = oracle.attn_fwd(q.numpy(), k.numpy(), v.numpy(), scale, causal=causal)
    dq, dk, dv = oracle.attn_bwd(q.numpy(), k.numpy(), v.numpy(), do.numpy(), scale, causal=causal)
    return o, lse, dq, dk, dv


@pytest.mark.parametrize("world", [1, 2, 4])
@pytest.mark.parametrize("causal", [False, True])
def test_layout_round_trip_and_balance(world, causal):
    S = 32
    owned = [ring.owned_positions(S, world, r, causal) for r in range(world)]
    assert sorted(torch.cat(owned).tolist()) == list(range(S))
    x = torch.arange(2 * 3 * S * 4, dtype=torch.float32).view(2, 3, S, 4)
    parts = [ring.shard_sequence(x, world, r, causal) for r in range(world)]
    assert torch.equal(ring.unshard_sequence(parts, causal), x)
    if causal:
        # every rank computes the same number of unmasked (query, key) pairs at every step
        L = S // world
        for step in range(world):
            work = set()
            for r in range(world):
                (_, qn), (_, kn), cz = ring.block_plan(r, (r - step) % world, L, True)
                work.add(qn * (qn + 1) // 2 if cz else qn * kn)
            assert len(work) == 1
    with pytest.raises(ValueError):
        ring.owned_positions(30, 4, 0, True)


@pytest.mark.parametrize("world", [1, 2, 4])
@pytest.mark.parametrize("causal", [False, True])
def test_emulated_schedule_matches_the_oracle(world, causal):
    B, H, S, D = 1, 2, 32, 8
    scale = 1 / math.sqrt(D)
    q, k, v, do = _problem(B, H, S, D, 3)
    ops = NumpyOps(scale)
    sh = lambda x: [ring.shard_sequence(x, world, r, causal) for r in range(world)]
    qs, ks, vs, dos = sh(q), sh(k), sh(v), sh(do)
    fwd = ring.ring_attention_fwd_emulated(ops, qs, ks, vs, causal)
    o = ring.unshard_sequence([f[0] for f in fwd], causal)
    lse = ring.unshard_sequence([f[1] for f in fwd], causal)
    ro, rlse, rdq, rdk, rdv = _oracle(q, k, v, do, scale, causal)
    assert np.abs(o.numpy() - ro).max() < 2e-6 and np.abs(lse.numpy() - rlse).max() < 2e-6
    bwd = ring.ring_attention_bwd_emulated(ops, qs, ks, vs, [f[0] for f in fwd], [f[1] for f in fwd], dos, causal)
    for i, ref in enumerate((rdq, rdk, rdv)):
        got = ring.unshard_sequence([b[i] for b in bwd], causal)
        assert np.abs(got.numpy() - ref).max() < 5e-6


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _ring_worker(rank, world, port, causal, half, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        B, H, S, D = 1, 2, 32, 8
        scale = 1 / math.sqrt(D)
        q, k, v, do = _problem(B, H, S, D, 5)               # every rank draws the same whole problem
        if half:                                            # 16-bit storage: the hop home carries rounded gradients
            q, k, v, do = (x.half() for x in (q, k, v, do))
        mine = [ring.shard_sequence(x, world, rank, causal) for x in (q, k, v, do)]
        ops = NumpyOps(scale)
        o, lse = ring.ring_attention_fwd(ops, *mine[:3], rank, world, causal)
        dq, dk, dv = ring.ring_attention_bwd(ops, *mine[:3], o, lse, mine[3], rank, world, causal)
        ref = _oracle(q.float(), k.float(), v.float(), do.float(), scale, causal)
        idx = ring.owned_positions(S, world, rank, causal).numpy()
        assert dq.dtype == q.dtype and dk.dtype == q.dtype and o.dtype == q.dtype
        errs = [float(np.abs(got.float().numpy() - r[:, :, idx]).max())
                for got, r in zip((o, lse, dq, dk, dv), ref)]
        out[rank] = max(errs)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("causal,half", [(False, False), (True, False), (True, True)])
def test_two_gloo_ranks_exchange_their_slices(causal, half):
    world = 2
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_ring_worker, args=(world, _free_port(), causal, half, out), nprocs=world, join=True)
    assert all(out[r] < (3e-3 if half else 5e-6) for r in range(world))


@pytest.mark.gpu
@pytest.mark.parametrize("world,causal,S,dtype", [(2, True, 1024, torch.bfloat16), (4, True, 2048, torch.bfloat16),
                                                  (2, False, 512, torch.bfloat16), (2, True, 64, torch.float32),
                                                  (4, False, 96, torch.float32)])
def test_cuda_kernels_under_the_emulated_schedule(world, causal, S, dtype):
    from cuda_ltc_b200 import Context
    ctx = Context()
    B, H, D = 1, 2, 64
    scale = 1 / math.sqrt(D)
    q, k, v, do = (x.to(dtype) for x in _problem(B, H, S, D, 11))
    ref = _oracle(q.float(), k.float(), v.float(), do.float(), scale, causal)
    from cuda_ltc_b200 import _lib
    ops = ring.CudaOps(ctx, scale, _lib.MODE_FP32 if dtype == torch.float32 else _lib.MODE_AUTO)
    sh = lambda x: [ring.shard_sequence(x.cuda(), world, r, causal) for r in range(world)]
    qs, ks, vs, dos = sh(q), sh(k), sh(v), sh(do)
    fwd = ring.ring_attention_fwd_emulated(ops, qs, ks, vs, causal)
    bwd = ring.ring_attention_bwd_emulated(ops, qs, ks, vs, [f[0] for f in fwd], [f[1] for f in fwd], dos, causal)
    got = [ring.unshard_sequence([f[0] for f in fwd], causal), ring.unshard_sequence([f[1] for f in fwd], causal)]
    got += [ring.unshard_sequence([b[i] for b in bwd], causal) for i in range(3)]
    tol = 2e-3 if dtype == torch.bfloat16 else 2e-5
    for g_, r in zip(got, ref):
        g_ = g_.float().cpu().numpy()
        if dtype == torch.bfloat16:
            # outputs are rounded to bf16 on the way out: compare with that rounding's own step allowed
            assert np.abs(g_ - r).max() < tol + np.abs(r).max() * 2 ** -8
            assert np.linalg.norm(g_ - r) / np.linalg.norm(r) < 5e-3
        else:
            assert np.abs(g_ - r).max() < tol
    assert ctx.device_status() == 0


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_merge_and_accumulate_kernels(dtype):
    """ltca_attn_merge / ltca_accumulate_rows on a row range, rows without a visible key, and argument errors."""
    from cuda_ltc_b200 import Context
    from cuda_ltc_b200.api import LtcaError
    ctx = Context()
    B, H, S, D, s0, n = 2, 3, 40, 64, 8, 24
    g = torch.Generator(device="cuda").manual_seed(2)
    o_acc = torch.randn((B, H, S, D), generator=g, device="cuda")
    lse_acc = torch.randn((B, H, S), generator=g, device="cuda")
    lse_acc[0, 0, s0 + 1] = float("-inf")                    # nothing accumulated yet on this row
    o_blk = torch.randn((B, H, n, D), generator=g, device="cuda").to(dtype)
    lse_blk = torch.randn((B, H, n), generator=g, device="cuda")
    lse_blk[1, 2, 3] = float("-inf")                         # this row saw no key in the block
    want_o, want_l = o_acc.double().clone(), lse_acc.double().clone()
    la, lb = want_l[:, :, s0:s0 + n], lse_blk.double()
    new = torch.logaddexp(la, lb)
    wa = torch.where(torch.isinf(la) & (la < 0), torch.zeros_like(la), torch.exp(la - new))
    wb = torch.where(torch.isinf(lb) & (lb < 0), torch.zeros_like(lb), torch.exp(lb - new))
    want_o[:, :, s0:s0 + n] = want_o[:, :, s0:s0 + n] * wa[..., None] + o_blk.double() * wb[..., None]
    want_l[:, :, s0:s0 + n] = new
    ctx.attn_merge(o_acc, lse_acc, o_blk, lse_blk, s0)
    assert torch.allclose(o_acc.double(), want_o, atol=2e-5, rtol=1e-5)
    assert torch.allclose(lse_acc.double(), want_l, atol=1e-5)
    assert torch.equal(o_acc[1, 2, s0 + 3].double(), want_o[1, 2, s0 + 3])     # untouched row: same bits

    acc = torch.randn((B, H, S, D), generator=g, device="cuda")
    part = torch.randn((B, H, n, D), generator=g, device="cuda").to(dtype)
    want = acc.clone()
    want[:, :, s0:s0 + n] += part.float()
    ctx.accumulate_rows(acc, part, s0)
    assert torch.equal(acc, want)

    with pytest.raises(LtcaError):
        ctx.accumulate_rows(acc, part, S - n + 1)            # the range runs past the accumulator
    with pytest.raises(LtcaError):
        ctx.attn_merge(o_acc, lse_acc, o_blk, lse_blk, S)
    assert ctx.device_status() == 0


def _nccl_ring_worker(rank, world, port, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from cuda_ltc_b200 import Context
        ctx = Context(rank)
        B, H, S, D = 1, 4, 2048, 64
        scale = 1 / math.sqrt(D)
        q, k, v, do = (x.bfloat16() for x in _problem(B, H, S, D, 21))     # same whole problem on every rank
        ref = _oracle(q.float(), k.float(), v.float(), do.float(), scale, True)
        mine = [ring.shard_sequence(x.cuda(), world, rank, True) for x in (q, k, v, do)]
        ops, cache = ring.CudaOps(ctx, scale), {}
        worst, detail = 0.0, []
        for _ in range(2):                                   # the second pass runs on reused buffers
            o, lse = ring.ring_attention_fwd(ops, *mine[:3], rank, world, True, cache=cache)
            dq, dk, dv = ring.ring_attention_bwd(ops, *mine[:3], o, lse, mine[3], rank, world, True, cache=cache)
            torch.cuda.synchronize()
            idx = ring.owned_positions(S, world, rank, True).numpy()
            for got, r in zip((o, lse, dq, dk, dv), ref):
                r = r[:, :, idx]
                err = np.abs(got.float().cpu().numpy() - r).max() / (2e-3 + np.abs(r).max() * 2 ** -8)
                detail.append(round(float(err), 3))
                worst = max(worst, float(err))
        out[rank] = (worst, ctx.device_status(), detail)
    finally:
        dist.destroy_process_group()


@pytest.mark.gpu
@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_gpu_ranks_exchange_over_nccl():
    """The real transport: two processes, one GPU each, NCCL point-to-point hops, buffers reused across
    passes; every rank's slice of O, lse, dQ, dK, dV against the oracle on the whole sequence."""
    world = 2
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_nccl_ring_worker, args=(world, _free_port(), out), nprocs=world, join=True)
    for r in range(world):
        worst, status, detail = out[r]
        # unit = 2e-3 + one bf16 step of the largest element; every pair's partial result leaves the kernels
        # rounded to bf16 and the sum is rounded once more, so up to 1.5 units are rounding alone
        assert worst < 1.5 and status == 0, f"rank {r}: error / tolerance per tensor and pass {detail}"


def _dead_rank_worker(rank, world, port, out):
    """Rank 1 joins the group and then leaves between steps without ever sending; rank 0 starts the ring."""
    import datetime
    import time
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=5))
    dist.barrier()                                         # both ranks are up: the failure happens after this
    if rank == 1:
        out[rank] = "left"
        os._exit(0)                                        # no goodbye: the peer learns of it from the transport
    B, H, S, D = 1, 2, 32, 8
    q, k, v, _ = _problem(B, H, S, D, 5)
    mine = [ring.shard_sequence(x, world, rank, True) for x in (q, k, v)]
    t0 = time.time()
    try:
        ring.ring_attention_fwd(NumpyOps(1 / math.sqrt(D)), *mine, rank, world, True)
        out[rank] = "finished"                             # must not happen: half of the keys never arrived
    except Exception as e:                                 # the hop's wait() raises: time-out or closed connection
        out[rank] = ("error", type(e).__name__, time.time() - t0)
    os._exit(0)


def test_a_rank_that_never_sends_ends_the_hop_with_an_error_not_a_hang():
    """Failure detection of the ring, on the host: a peer that disappears between steps turns the next hop's
    wait into an exception within the process group's time-out (5 s here); nothing spins for ever."""
    world = 2
    mgr = mp.Manager()
    out = mgr.dict()
    ctx = mp.get_context("spawn")
    port = _free_port()
    procs = [ctx.Process(target=_dead_rank_worker, args=(r, world, port, out)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(60)
    alive = [p for p in procs if p.is_alive()]
    for p in alive:
        p.kill()
    assert not alive, "a rank hung instead of failing"
    assert out.get(1) == "left"
    assert isinstance(out.get(0), tuple) and out[0][0] == "error", out.get(0)
    assert out[0][2] < 30
