"""Host-side logic of the multi-GPU run, on CPU: the partition of (batch, head) pairs and the
max-over-ranks reduction, the latter with two gloo ranks."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from cuda_ltc_b200.shard import batch_slices, reduce_max, unit_range


@pytest.mark.parametrize("n,world", [(128, 1), (128, 2), (128, 8), (8, 8), (5, 4), (3, 8), (0, 2)])
def test_every_unit_has_one_owner(n, world):
    seen = []
    for r in range(world):
        seen.extend(unit_range(n, world, r))
    assert seen == list(range(n))
    sizes = [len(unit_range(n, world, r)) for r in range(world)]
    assert max(sizes) - min(sizes) <= 1


def test_batch_slices_cover_the_rank_range():
    B, H, world = 3, 4, 5
    pairs = []
    for r in range(world):
        for b, h0, h1 in batch_slices(B, H, world, r):
            assert 0 <= h0 < h1 <= H
            pairs.extend((b, h) for h in range(h0, h1))
    assert pairs == [(b, h) for b in range(B) for h in range(H)]


def test_bad_rank_is_rejected():
    with pytest.raises(ValueError):
        unit_range(8, 2, 2)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        # each rank reports its own "time" and the units it owns; the reduction must give the slowest rank
        mine = unit_range(10, world, rank)
        red = reduce_max([1.0 + rank, float(len(mine))])
        total = torch.tensor([float(len(mine))])
        dist.all_reduce(total)
        out[rank] = (red, total.item())
    finally:
        dist.destroy_process_group()


def test_max_over_ranks_with_two_gloo_ranks():
    world = 2
    port = _free_port()
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_worker, args=(world, port, out), nprocs=world, join=True)
    for r in range(world):
        red, total = out[r]
        assert red == [2.0, 5.0]
        assert total == 10.0


def _module_worker(rank, world, port, out):
    """Each rank differentiates the module on its own sequences; the weight gradients are summed."""
    import numpy as np
    import oracle
    from cuda_ltc_b200.shard import sum_weight_grads
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        B, S, E, H = 4, 8, 16, 2
        rng = np.random.default_rng(7)
        x = rng.standard_normal((B, S, E))
        dy = rng.standard_normal((B, S, E))
        ws = [rng.standard_normal((E, E)) * 0.2 for _ in range(4)]
        mine = unit_range(B, world, rank)
        sl = slice(mine.start, mine.stop)
        kw = dict(scale=(E // H) ** -0.5, causal=True, time_major=False)
        part = oracle.tsa_bwd(x[sl].reshape(-1, E), *ws, dy[sl].reshape(-1, E), len(mine), S, H, E // H, **kw)
        grads = [torch.from_numpy(np.ascontiguousarray(g)) for g in part[1:5]]
        if rank == 0:
            # back-to-back views of one allocation are summed in place, separate tensors through a bucket
            flat = torch.cat([g.reshape(-1) for g in grads])
            views, off = [], 0
            for g in grads:
                views.append(flat[off:off + g.numel()].view(g.shape))
                off += g.numel()
            grads = views
        handle = sum_weight_grads(grads, async_op=True)
        done = handle.wait()
        assert len(done) == 4 and all(a is b for a, b in zip(done, grads))
        full = oracle.tsa_bwd(x.reshape(-1, E), *ws, dy.reshape(-1, E), B, S, H, E // H, **kw)
        err = max(float(np.abs(g.numpy() - f).max()) for g, f in zip(grads, full[1:5]))
        # the input gradient of the rank's rows needs no exchange at all
        dx_err = float(np.abs(part[0] - full[0].reshape(B, S, E)[sl].reshape(-1, E)).max())
        out[rank] = (err, dx_err)
    finally:
        dist.destroy_process_group()


def test_module_weight_gradients_sum_over_two_gloo_ranks():
    world = 2
    port = _free_port()
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_module_worker, args=(world, port, out), nprocs=world, join=True)
    for r in range(world):
        err, dx_err = out[r]
        assert err < 1e-10 and dx_err < 1e-10


def test_weight_gradient_sum_without_a_group_is_the_identity():
    from cuda_ltc_b200.shard import sum_weight_grads
    g = [torch.ones(3, 3), None, torch.full((2,), 2.0)]
    got = sum_weight_grads(g)
    assert len(got) == 2 and torch.equal(got[0], torch.ones(3, 3)) and torch.equal(got[1], torch.full((2,), 2.0))
    waited = sum_weight_grads(g, async_op=True).wait()       # the handle gives the same gradients back
    assert len(waited) == 2 and waited[0] is got[0] and waited[1] is got[1]
