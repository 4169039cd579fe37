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
