"""GPU tests of the small entry points beside the attention kernels, through the C ABI: tensor add, finite
check, LayerNorm, fp32 <-> bf16 conversion (what the reference's addTensors / validateGradients / applyLayerNorm
do: src/cuda_tensor_utils.cu:6-41, src/ml/cudnn_time_self_attention.cu:9-68, :496-508), the bounded-wait
self-test, and contexts on two devices of one process."""
import numpy as np
import pytest
import torch

from cuda_ltc_b200 import _lib
from util import bf16_round, max_abs, randn

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n,offset", [(1, 0), (7, 0), (4096, 0), (1000003, 0), (1001, 1)])
def test_add_tensors(ctx, n, offset):
    a, b = randn((n + offset,), 1), randn((n + offset,), 2)
    ta, tb = torch.from_numpy(a).cuda()[offset:], torch.from_numpy(b).cuda()[offset:]     # offset 1: unaligned path
    out = ctx.add_tensors(ta, tb)
    assert np.array_equal(out.cpu().numpy(), a[offset:] + b[offset:])                      # one fp32 add: exact
    ctx.add_tensors(ta, tb, out=ta)                                                        # in place
    assert np.array_equal(ta.cpu().numpy(), a[offset:] + b[offset:])


def test_validate_finite(ctx):
    x = torch.from_numpy(randn((100003,), 3)).cuda()
    assert ctx.validate_finite(x)
    for bad, where in ((float("nan"), 0), (float("inf"), 100002), (float("-inf"), 51234)):
        y = x.clone()
        y[where] = bad
        assert not ctx.validate_finite(y)
    assert ctx.validate_finite(x[:0])                       # nothing to check
    big = torch.full((1000,), 3.0e38, device="cuda")        # large but finite
    assert ctx.validate_finite(big)


@pytest.mark.parametrize("rows,E", [(1, 8), (33, 64), (1000, 512), (7, 100)])
def test_layer_norm(ctx, rows, E):
    x = randn((rows, E), 4) * 3.0 + 0.5
    gamma = (1.0 + 0.1 * randn((E,), 5)).astype(np.float32)
    beta = (0.1 * randn((E,), 6)).astype(np.float32)
    x64 = x.astype(np.float64)
    mean = x64.mean(axis=1, keepdims=True)
    var = ((x64 - mean) ** 2).mean(axis=1, keepdims=True)          # biased, as the reference's kernel
    ref = (x64 - mean) / np.sqrt(var + 1e-5) * gamma + beta
    t = torch.from_numpy(x.copy()).cuda()
    ctx.layer_norm_(t, torch.from_numpy(gamma).cuda(), torch.from_numpy(beta).cuda())
    assert max_abs(t.cpu().numpy(), ref) < 1e-5 * max(1.0, np.abs(ref).max())
    t = torch.from_numpy(x.copy()).cuda()
    ctx.layer_norm_(t)                                             # no scale / shift
    assert max_abs(t.cpu().numpy(), (x64 - mean) / np.sqrt(var + 1e-5)) < 1e-5 * 5


def test_bf16_conversions(ctx):
    x = np.concatenate([randn((100001,), 7) * 10.0,
                        np.array([0.0, -0.0, 1.0, 1.00390625, 1.005859375, 3.0e38, -1e-40, 65504.0], np.float32)])
    t = torch.from_numpy(x).cuda()
    b = ctx.to_bf16(t)
    assert np.array_equal(b.float().cpu().numpy(), bf16_round(x))          # round to nearest even, bit for bit
    back = ctx.to_f32(b)
    assert np.array_equal(back.cpu().numpy(), bf16_round(x))               # widening is exact


def test_bounded_wait_gives_up_and_reports(ctx):
    """A wait whose barrier never completes must end by itself, set the time-out bit and the code of the
    barrier in the status word, and leave the context usable."""
    torch.cuda.synchronize()
    assert ctx.device_status() == 0
    ctx.selftest_bounded_wait(20000)                                       # 20 ms instead of the kernels' 2 s
    status = ctx.device_status()                                           # synchronises the stream
    assert status & 1, hex(status)
    assert (status >> 8) & 0xffff == 0x7f
    assert ctx.device_status() == 0                                        # read-and-clear
    q = torch.from_numpy(randn((1, 2, 128, 64), 8) * 0.5).cuda().bfloat16()
    o, _ = ctx.attn_fwd(q, q, q, causal=True, mode=_lib.MODE_BF16)         # the context still works
    torch.cuda.synchronize()
    assert torch.isfinite(o.float()).all() and ctx.device_status() == 0


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs in one process")
def test_contexts_on_two_devices_of_one_process():
    """Every kernel that opts in to large dynamic shared memory must do so on each device it runs on."""
    import cuda_ltc_b200 as ltc
    outs = []
    for dev in (0, 1):
        with torch.cuda.device(dev):
            c = ltc.Context(dev)
            g = torch.Generator(device=f"cuda:{dev}").manual_seed(9)
            q, k, v, do = ((torch.randn((1, 2, 640, 64), generator=g, device=f"cuda:{dev}") * 0.5).bfloat16()
                           for _ in range(4))
            o, lse = c.attn_fwd(q, k, v, causal=True, mode=_lib.MODE_BF16)          # persistent 4-tile kernel
            o2, _ = c.attn_fwd(q[:, :, :200], k, v, mode=_lib.MODE_BF16)             # 2-tile kernel
            grads = c.attn_bwd(q, k, v, o, lse, do, causal=True)
            qf = q.float()
            of, lf = c.attn_fwd(qf, k.float(), v.float(), causal=True, mode=_lib.MODE_FP32)
            torch.cuda.synchronize(dev)
            assert c.device_status() == 0
            outs.append([t.cpu() for t in (o, o2, *grads, of)])
            c.close()
    for a, b in zip(*outs):
        assert torch.equal(a, b)
