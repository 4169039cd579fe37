"""Module-level data parallelism on real GPUs: two NCCL ranks, each differentiating the module on its own
sequences, sum their weight gradients with one collective; the result must equal the gradients of the whole
batch computed on one GPU.  Skipped where fewer than two GPUs are visible."""
import math
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from cuda_ltc_b200 import Context, _lib
        from cuda_ltc_b200.shard import sum_weight_grads, unit_range
        ctx = Context(rank)
        B, S, E, H, W = 8, 128, 256, 4, 64
        g = torch.Generator().manual_seed(9)                 # the same whole problem on every rank
        x = torch.randn((B, S, E), generator=g).cuda()
        dy = torch.randn((B, S, E), generator=g).cuda()
        lim = math.sqrt(6.0 / (2 * E))
        ws = [((torch.rand((E, H * W), generator=g) * 2 - 1) * lim).cuda() for _ in range(3)]
        wo = ((torch.rand((H * W, E), generator=g) * 2 - 1) * lim).cuda()
        kw = dict(scale=1 / math.sqrt(W), causal=True, time_major=False, mode=_lib.MODE_BF16)
        whole = ctx.tsa_bwd(x.view(-1, E), *ws, wo, dy.view(-1, E), B, S, H, W, **kw)
        mine = unit_range(B, world, rank)
        sl = slice(mine.start, mine.stop)
        part = ctx.tsa_bwd(x[sl].reshape(-1, E), *ws, wo, dy[sl].reshape(-1, E), len(mine), S, H, W, **kw)
        sum_weight_grads(part[1:])
        torch.cuda.synchronize()
        errs = [float((a - b).norm() / b.norm()) for a, b in zip(part[1:], whole[1:])]
        dx_same = bool(torch.equal(part[0], whole[0].view(B, S, E)[sl].reshape(-1, E)))
        out[rank] = (max(errs), dx_same, ctx.device_status())
    finally:
        dist.destroy_process_group()


@pytest.mark.gpu
@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_weight_gradients_summed_over_two_nccl_ranks():
    world = 2
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), out), nprocs=world, join=True)
    for r in range(world):
        err, dx_same, status = out[r]
        # the halves are summed in another order than the whole batch's contraction: fp32 rounding only
        assert err < 1e-4 and status == 0, (r, err)
        assert dx_same, "the input gradient of a rank's sequences must not depend on the partition"
