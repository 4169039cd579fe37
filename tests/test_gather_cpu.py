"""Sequence sharding with gathered K/V (cuda_ltc_b200.gather): two gloo ranks on the CPU exchange their slices
through torch.distributed collectives, the arithmetic of every block is an fp64 stand-in for the kernels with the
kernels' causal rule (key j visible to query i iff j <= i + Sk - Sq), and the result equals attention over the whole
sequence."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp


class NumpyOps:
    def __init__(self, scale):
        self.scale = scale

    def _scores(self, q, k, causal):
        s = np.einsum("bhid,bhjd->bhij", q.numpy().astype(np.float64), k.numpy().astype(np.float64)) * self.scale
        if causal:
            off = s.shape[3] - s.shape[2]
            i, j = np.arange(s.shape[2])[:, None], np.arange(s.shape[3])[None, :]
            s = np.where(j <= i + off, s, -np.inf)
        return s

    def block_fwd(self, q, k, v, causal, out=None, lse=None):
        s = self._scores(q, k, causal)
        m = s.max(-1, keepdims=True)
        p = np.exp(s - m)
        l = p.sum(-1, keepdims=True)
        out.copy_(torch.from_numpy(np.einsum("bhij,bhjd->bhid", p / l, v.numpy().astype(np.float64))))
        lse.copy_(torch.from_numpy((m + np.log(l))[..., 0]))
        return out, lse

    def block_bwd(self, q, k, v, o, lse, dout, causal, dq=None, dk=None, dv=None):
        s = self._scores(q, k, causal)
        p = np.exp(s - lse.numpy().astype(np.float64)[..., None])
        do = dout.numpy().astype(np.float64)
        dp = np.einsum("bhid,bhjd->bhij", do, v.numpy().astype(np.float64))
        delta = (do * o.numpy().astype(np.float64)).sum(-1, keepdims=True)
        ds = p * (dp - delta) * self.scale
        dq.copy_(torch.from_numpy(np.einsum("bhij,bhjd->bhid", ds, k.numpy().astype(np.float64))))
        dk.copy_(torch.from_numpy(np.einsum("bhij,bhid->bhjd", ds, q.numpy().astype(np.float64))))
        dv.copy_(torch.from_numpy(np.einsum("bhij,bhid->bhjd", p, do)))
        return dq, dk, dv

    def accumulate(self, acc, part, s0):
        acc[:, :, s0:s0 + part.shape[2]] += part.float()


def _whole(q, k, v, do, scale, causal):
    ops = NumpyOps(scale)
    o, lse = torch.empty_like(q), torch.empty(q.shape[:3], dtype=q.dtype)
    ops.block_fwd(q, k, v, causal, out=o, lse=lse)
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    ops.block_bwd(q, k, v, o, lse, do, causal, dq=dq, dk=dk, dv=dv)
    return o, dq, dk, dv


def _rank_main(rank, world, port, causal, ret):
    import torch.distributed as dist
    from cuda_ltc_b200 import gather, ring
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(7)
        B, H, S, D = 2, 2, 24, 8
        q, k, v, do = (torch.randn((B, H, S, D), generator=g, dtype=torch.float64) for _ in range(4))
        scale = D ** -0.5
        want = _whole(q, k, v, do, scale, causal)
        ops = NumpyOps(scale)
        sl = lambda x: ring.shard_sequence(x, world, rank, causal)
        cache = {}
        for _ in range(2):                                   # the second pass runs on reused buffers
            o, lse, kf, vf = gather.gathered_attention_fwd(ops, sl(q), sl(k), sl(v), rank, world, causal, cache=cache)
            dq, dk, dv = gather.gathered_attention_bwd(ops, sl(q), kf, vf, o, lse, sl(do), rank, world, causal,
                                                       cache=cache)
        err = max(float((a - sl(b)).abs().max()) for a, b in zip((o, dq, dk, dv), want))
        ret[rank] = err
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("causal", [False, True])
def test_two_gloo_ranks_equal_the_whole_sequence(causal):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    procs = [ctx.Process(target=_rank_main, args=(r, 2, port, causal, ret)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert len(ret) == 2 and max(ret.values()) < 1e-5        # dk / dv travel as fp32


def test_query_blocks_cover_the_causal_triangle_evenly():
    from cuda_ltc_b200.gather import _query_blocks
    world, c = 4, 3
    work = []
    for r in range(world):
        blocks = _query_blocks(r, world, 2 * c, True)
        assert [b[:2] for b in blocks] == [(0, c), (c, c)]
        assert blocks[0][2] == (r + 1) * c and blocks[1][2] == (2 * world - r) * c
        work.append(sum(n * nk for _, n, nk in blocks))
    assert len(set(work)) == 1                               # the same number of scores on every rank
    assert _query_blocks(1, 4, 5, False) == [(0, 5, 20)]


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("world", [1, 2, 4])
def test_shares_land_with_the_rank_that_owns_the_key(world, causal):
    """_add_shares against the layout's own definition (ring.owned_positions), for every prefix length a rank's
    calls can have."""
    from cuda_ltc_b200 import gather, ring
    B, H, D, c = 2, 3, 4, 5
    L = 2 * c if causal else c
    S = world * L
    g = torch.Generator().manual_seed(3)
    prefixes = sorted({nk for r in range(world) for _, _, nk in gather._query_blocks(r, world, L, causal)})
    for nk in prefixes:
        part = torch.randn((B, H, nk, D), generator=g)
        send = torch.zeros((world, 2, B, H, L, D))
        gather._add_shares(send, 1, part, world, L, causal)
        full = torch.zeros((B, H, S, D))
        full[:, :, :nk] = part
        for r in range(world):
            want = full.index_select(2, ring.owned_positions(S, world, r, causal))
            assert torch.equal(send[r, 1], want), (nk, r)
        assert float(send[:, 0].abs().max()) == 0.0


@pytest.mark.parametrize("causal", [False, True])
def test_gathered_slices_come_back_in_sequence_order(causal):
    """The reordering inside gather_sequence (no collective at world 1; here the gathered block is handed in
    directly) inverts ring.shard_sequence for every rank count."""
    from cuda_ltc_b200 import gather, ring
    B, H, D = 2, 2, 3
    for world in (2, 3, 4):
        S = world * 6
        x = torch.arange(B * H * S * D, dtype=torch.float32).view(B, H, S, D)
        flat = torch.stack([ring.shard_sequence(x, world, r, causal) for r in range(world)])

        class _FakeDist:
            @staticmethod
            def all_gather_into_tensor(out, inp, group=None):
                out.copy_(flat.view(-1))
        old = gather._dist
        gather._dist = lambda: _FakeDist
        try:
            full = gather.gather_sequence(flat[0], world, causal)
        finally:
            gather._dist = old
        assert torch.equal(full, x)
