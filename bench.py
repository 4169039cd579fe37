#!/usr/bin/env python
"""Benchmark of the attention hot path (forward + backward of the attention core).

Workload (BASELINE.json configs[2], the configuration the headline target is quoted on):
B=8 H=16 S=4096 D=64, causal, bf16 storage with fp32 accumulation, Q/K/V/dO = 0.5*N(0,1) from a
seed.  A step is one forward and one backward over the whole batch.  With N GPUs every rank
processes its own B=8 slice of a global batch of 8*N sequences (batch x head partition, no
collective on the data path), so scaling is weak.

    python bench.py --gpus 1 --steps 20 --warmup 3
    python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N ...
    python bench.py --impl reference          # CPU arm: the fp64 oracle port on the host cores

Prints ONE JSON line (rank 0).  FLOP accounting: forward = 4*B*H*S*S*D/2 (causal half),
backward = 2.5x forward; recomputation and softmax are not counted.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

CFG = dict(B=8, H=16, S=4096, D=64, causal=True)
SEED = 20241


def flops_fwd(B, H, S, D, causal=True):
    return 4.0 * B * H * S * S * D * (0.5 if causal else 1.0)


def measured_peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return json.load(f), "measured"
    except Exception:
        return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML while the timed region runs."""

    def __init__(self, index: int):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self._nv = None

    def _run(self):
        nv = self._nv
        names = {
            "hw_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwSlowdown", 0x8),
            "hw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40),
            "sw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20),
            "sw_power_cap": getattr(nv, "nvmlClocksThrottleReasonSwPowerCap", 0x4),
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM))
                r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._h)
                for n, bit in names.items():
                    if r & bit:
                        self.reasons.add(n)
            except Exception:
                pass
            self._stop.wait(0.02)

    def start(self):
        if self._nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2] if s else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons)}


def physical_gpu_index(local_rank: int) -> int:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local_rank])
        except Exception:
            return local_rank
    return local_rank


def run_cpu_sample(n_bh: int, threads: int | None = None):
    """fp64 oracle forward + backward on `n_bh` (batch, head) pairs of the workload."""
    import numpy as np
    import oracle
    if threads:
        oracle.set_num_threads(threads)
    S, D = CFG["S"], CFG["D"]
    rng = np.random.default_rng(SEED)
    q, k, v, do = ((rng.standard_normal((1, n_bh, S, D)) * 0.5).astype(np.float32) for _ in range(4))
    t0 = time.perf_counter()
    oracle.attn_fwd(q, k, v, 1.0 / math.sqrt(D), True)
    oracle.attn_bwd(q, k, v, do, 1.0 / math.sqrt(D), True)
    dt = time.perf_counter() - t0
    fl = 3.5 * flops_fwd(1, n_bh, S, D)
    return fl / dt / 1e12, dt, oracle.num_threads()


def reference_arm(args):
    """CPU arm: the reference has no CPU implementation of this path (all of it is CUDA and its
    own kernels cannot run this configuration), so the timed code is the repository's fp64
    OpenMP port of the same arithmetic, on all host threads, on a bounded sample per step."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    n_bh = max(8, min(cores, 64))
    for _ in range(args.warmup if args.warmup < 2 else 1):
        run_cpu_sample(max(2, n_bh // 4))
    t_total, fl_total = 0.0, 0.0
    threads = 1
    for _ in range(args.steps):
        tf, dt, threads = run_cpu_sample(n_bh)
        t_total += dt
        fl_total += tf * dt
    value = fl_total / t_total
    sample = f"{n_bh} of {CFG['B'] * CFG['H']} (batch, head) pairs per step, forward + backward, fp64"
    line = {
        "impl": "reference", "metric": "attention fwd+bwd TFLOP/s", "value": value, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1000.0 * t_total / max(1, args.steps), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f64", "data": "synthetic",
        "config": workload_config(args.gpus),
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def workload_config(n_gpus):
    return {"workload": f"attention core fwd+bwd, B={CFG['B']} H=16 S=4096 D=64 causal, bf16 storage / fp32 "
                        "accumulate (BASELINE configs[2]" + ("" if CFG["B"] == 8 else ", reduced batch") + "); per GPU",
            "global_batch": CFG["B"] * n_gpus, "heads": CFG["H"], "seq_len": CFG["S"], "head_dim": CFG["D"],
            "parallelism": f"batch x head partition over {n_gpus} GPU(s), no collective",
            "l2": f"inputs ({32 * CFG['B']} MB per step) exceed the 126 MB L2; no explicit flush"}


def module_measurement(args):
    """TimeSelfAttention forward and backward (with the recomputed forward) at B=32 S=256 E=512 H=8 per GPU,
    head width 64, causal; with several ranks the weight gradients are summed over them after each
    backward.  Back-to-back calls between CUDA events; an L2 flush is not needed for a figure that is dominated
    by eleven GEMMs over 16 MB activations.  Rank 0 prints one JSON line (maximum over the ranks' times)."""
    import math
    import torch
    import torch.distributed as dist
    import cuda_ltc_b200 as ltc
    from cuda_ltc_b200 import _lib
    from cuda_ltc_b200.shard import reduce_max, sum_weight_grads
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    ctx = ltc.Context(local_rank)
    B, S, E, H, W = 32, 256, 512, 8, 64                 # per rank: sequences are dealt out, weights replicated
    g = torch.Generator(device="cuda").manual_seed(SEED + rank)
    x = torch.randn((B * S, E), generator=g, device="cuda")
    dy = torch.randn((B * S, E), generator=g, device="cuda")
    gw = torch.Generator(device="cuda").manual_seed(SEED)
    lim = math.sqrt(6.0 / (2 * E))
    ws = [(torch.rand((E, H * W), generator=gw, device="cuda") * 2 - 1) * lim for _ in range(3)]
    wo = (torch.rand((H * W, E), generator=gw, device="cuda") * 2 - 1) * lim
    gamma, beta = torch.ones(E, device="cuda"), torch.zeros(E, device="cuda")
    kw = dict(scale=1 / math.sqrt(W), causal=True, time_major=False, mode=_lib.MODE_BF16)
    fwd = lambda: ctx.tsa_fwd(x, *ws, wo, B, S, H, W, gamma=gamma, beta=beta, **kw)

    def bwd():
        grads = ctx.tsa_bwd(x, *ws, wo, dy, B, S, H, W, **kw)
        sum_weight_grads(grads[1:])                     # one 4 MiB sum over the ranks; nothing at one rank
        return grads

    n, w = (1, 1) if args.profile else (max(5, args.steps), max(3, args.warmup))

    def timed(f):
        for _ in range(w):
            f()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            f()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / n

    f_ms, b_ms = reduce_max([timed(fwd), timed(bwd)])
    status = ctx.device_status()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if rank != 0:
        return
    rows = B * S * world
    gemm = 2.0 * rows * E * H * W                       # one projection
    core = 4.0 * B * world * H * S * S * W / 2
    print(json.dumps({"workload": "TimeSelfAttention module, B=32 per GPU, S=256 E=512 H=8 W=64 causal, "
                                  "tensor-pipe mode; weight gradients summed over the ranks",
                      "n_gpus": world,
                      "fwd_us": f_ms * 1e3, "bwd_incl_recompute_us": b_ms * 1e3,
                      "fwd_tflops": (4 * gemm + core) / f_ms / 1e9,
                      "bwd_tflops": (11 * gemm + 3.5 * core) / b_ms / 1e9,
                      "device_status": status}))


def model_step_measurement(args):
    """Attention's share of a model-shaped training step (BASELINE configs[4]: B=64, S=512, fp32).

    Only the attention module is this library's code.  Its neighbours in the reference's model
    (src/ml/ml_liquid_net.cu:146-170: PreConvBlock -> positional embedding -> projection ->
    TimeSelfAttention -> LTCBlock -> PolicyHead / ValueNet) are plain torch stand-ins of the same shapes,
    there to give the step its surrounding cost, not to reproduce those layers: a k=3 convolution 64 -> 512
    with LayerNorm and GELU, a learned positional table, a 512 x 512 projection, a recurrent cell of 256
    units stepped over the 512 positions with 6 semi-implicit ODE unfolds per position (the update rule of
    src/ml/ltc_cell.cu:59-106), and two linear heads (16 actions, 1 value) on the last state.
    The attention module's forward and backward are bracketed by CUDA events inside the step."""
    import math
    import torch
    import torch.nn.functional as F
    import cuda_ltc_b200 as ltc
    from cuda_ltc_b200 import _lib
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    ctx = ltc.Context(0)
    B, S, Cin, E, H, W, U, UNF, ACT = 64, 512, 64, 512, 8, 64, 256, 6, 16
    g = torch.Generator(device=dev).manual_seed(SEED)

    def param(*shape, fan):
        lim = math.sqrt(6.0 / fan)
        return ((torch.rand(shape, generator=g, device=dev) * 2 - 1) * lim).requires_grad_()

    conv_w, conv_b = param(E, Cin, 3, fan=Cin * 3 + E), torch.zeros(E, device=dev, requires_grad=True)
    ln_g, ln_b = torch.ones(E, device=dev, requires_grad=True), torch.zeros(E, device=dev, requires_grad=True)
    pos = (torch.randn((S, E), generator=g, device=dev) * 0.02).requires_grad_()
    proj_w = param(E, E, fan=2 * E)
    wq, wk, wv, wo = (param(E, E, fan=2 * E) for _ in range(4))
    a_gamma, a_beta = torch.ones(E, device=dev), torch.zeros(E, device=dev)
    w_in, w_rec = param(E, 4 * U, fan=E + U), param(U, 4 * U, fan=2 * U)
    b_gate = torch.zeros(4 * U, device=dev, requires_grad=True)
    tau = torch.ones(U, device=dev, requires_grad=True)
    a_vec = torch.ones(U, device=dev, requires_grad=True)
    pol_w, val_w = param(U, ACT, fan=U + ACT), param(U, 1, fan=U + 1)
    params = [conv_w, conv_b, ln_g, ln_b, pos, proj_w, wq, wk, wv, wo, w_in, w_rec, b_gate, tau, a_vec, pol_w,
              val_w]
    x_in = torch.randn((B, S, Cin), generator=g, device=dev)
    kw = dict(scale=1 / math.sqrt(W), causal=True, time_major=False, mode=_lib.MODE_BF16)
    attn_events = []
    # the forward keeps its intermediates for the backward (no recomputation inside the step)
    saved = ctx.tsa_saved_buffer(torch.empty((B * S, E), device=dev), wq, wk, wv, wo, B, S, H, W,
                                 mode=_lib.MODE_BF16, causal=True)

    class Attention(torch.autograd.Function):
        @staticmethod
        def forward(fctx, x, wq_, wk_, wv_, wo_):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            out = ctx.tsa_fwd(x, wq_, wk_, wv_, wo_, B, S, H, W, gamma=a_gamma, beta=a_beta, saved=saved, **kw)
            e1.record()
            attn_events.append((e0, e1))
            fctx.save_for_backward(x, wq_, wk_, wv_, wo_)
            return out

        @staticmethod
        def backward(fctx, dy):
            x, wq_, wk_, wv_, wo_ = fctx.saved_tensors
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            grads = ctx.tsa_bwd(x, wq_, wk_, wv_, wo_, dy.contiguous(), B, S, H, W, saved=saved,
                                reuse_forward=True, **kw)
            e1.record()
            attn_events.append((e0, e1))
            return grads

    def step(recurrent=True):
        h = F.conv1d(x_in.transpose(1, 2), conv_w, conv_b, padding=1).transpose(1, 2)
        h = F.gelu(F.layer_norm(h, (E,), ln_g, ln_b)) + pos
        h = (h.reshape(B * S, E) @ proj_w).contiguous()
        h = Attention.apply(h, wq, wk, wv, wo)
        gates_in = (h @ w_in + b_gate).view(B, S, 4 * U)
        state = torch.zeros((B, U), device=dev)
        dt = 1.0 / UNF
        for t in range(S if recurrent else 1):
            i_t, f_t, o_t, c_t = (gates_in[:, t] + state @ w_rec).chunk(4, dim=1)
            i_t, f_t, o_t, c_t = torch.sigmoid(i_t), torch.sigmoid(f_t), torch.sigmoid(o_t), torch.tanh(c_t)
            f_x = o_t * torch.tanh(f_t * c_t + i_t * torch.tanh(a_vec))
            for _ in range(UNF):
                state = (state + dt * f_x * a_vec) / (1.0 + dt * (1.0 / tau.clamp_min(1e-6) + f_x))
        loss = (state @ pol_w).square().mean() + (state @ val_w).square().mean()
        loss.backward()
        for p_ in params:
            p_.grad = None
        return loss

    n, w = (1, 1) if args.profile else (max(2, min(args.steps, 5)), 1)
    for _ in range(w):
        step()
    torch.cuda.synchronize()
    attn_events.clear()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(n):
        step()
    e1.record()
    torch.cuda.synchronize()
    step_ms = e0.elapsed_time(e1) / n
    attn_ms = sum(a.elapsed_time(b) for a, b in attn_events) / n
    # the same step with the recurrent cell run at one position only: what is left when the cell's
    # launch-bound loop over the positions is taken out
    step(False)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(n):
        step(False)
    e1.record()
    torch.cuda.synchronize()
    flat_ms = e0.elapsed_time(e1) / n
    print(json.dumps({"workload": "model-shaped step, B=64 S=512 fp32 (BASELINE configs[4]); attention module = this "
                                  "library (tensor-pipe mode), every other layer a torch stand-in of the same shape",
                      "step_ms": step_ms, "attention_ms": attn_ms, "attention_share": attn_ms / step_ms,
                      "step_one_recurrent_position_ms": flat_ms, "attention_share_there": attn_ms / flat_ms,
                      "steps": n, "recurrent_positions": S, "ode_unfolds": UNF,
                      "device_status": ctx.device_status()}))


def ring_measurement(args):
    """The long-sequence configuration with the SEQUENCE dealt out over the ranks (ring exchange of K/V,
    zig-zag causal layout) instead of the batch: total work is fixed (B=8 H=16 S=4096 D=64 causal bf16), each
    rank holds S / N positions.  Launch with one rank per GPU; rank 0 prints one JSON line with the
    maximum over the ranks' times.  A side measurement, not the bench line: the batch x head partition
    needs no exchange and is the headline."""
    import torch
    import torch.distributed as dist
    import cuda_ltc_b200 as ltc
    from cuda_ltc_b200 import ring
    from cuda_ltc_b200.shard import reduce_max
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    dev = torch.device("cuda", local_rank)
    ctx = ltc.Context(local_rank)
    B, H, S, D = CFG["B"], CFG["H"], args.seq_len or CFG["S"], CFG["D"]
    L = S // world
    g = torch.Generator(device=dev).manual_seed(SEED + rank)
    mk = lambda: (torch.randn((B, H, L, D), generator=g, device=dev) * 0.5).bfloat16()
    q, k, v, do = mk(), mk(), mk(), mk()
    ops = ring.CudaOps(ctx, comm_sms=args.comm_sms)
    cache = {}                                          # scratch and receive buffers live across the steps
    n, w = max(5, args.steps), max(3, args.warmup)

    def step():
        o, lse = ring.ring_attention_fwd(ops, q, k, v, rank, world, causal=True, cache=cache)
        ring.ring_attention_bwd(ops, q, k, v, o, lse, do, rank, world, causal=True, cache=cache)

    for _ in range(w):
        step()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
        torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(n):
        step()
    e1.record()
    torch.cuda.synchronize()
    ms = reduce_max([e0.elapsed_time(e1) / n])[0]
    status = ctx.device_status()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if rank != 0:
        return
    flops = 3.5 * 4.0 * B * H * S * S * D / 2
    print(json.dumps({"workload": f"attention fwd+bwd, B={B} H={H} S={S} D={D} causal bf16, sequence dealt out over "
                                  f"{world} GPU(s) with ring K/V exchange (strong scaling)",
                      "n_gpus": world, "ms_per_step": ms, "tflops_whole_job": flops / ms / 1e9,
                      "comm_sms": args.comm_sms if world > 1 else 0,
                      "kv_bytes_per_hop_per_gpu": 2 * B * H * L * D * 2,
                      "dkv_bytes_per_hop_per_gpu": 2 * B * H * L * D * 4, "device_status": status}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--batch", type=int, default=CFG["B"],
                    help="sequences per GPU; anything but the default is a reduced case for profiler captures")
    ap.add_argument("--profile", action="store_true",
                    help="profiler capture mode: 1 warm-up, 1 step, no end-to-end or CPU legs (not a bench value)")
    ap.add_argument("--seq-len", type=int, default=0, help="sequence length of the --ring measurement (default: the "
                                                           "bench configuration's)")
    ap.add_argument("--comm-sms", type=int, default=16,
                    help="--ring: SMs the attention kernels leave free for the exchange's copy kernels")
    ap.add_argument("--ring", action="store_true",
                    help="side measurement, not the bench line: the same problem with the sequence dealt out over "
                         "the ranks and K/V exchanged round a ring (launch one rank per GPU)")
    ap.add_argument("--model-step", action="store_true",
                    help="side measurement, not the bench line: attention's share of a step shaped like BASELINE "
                         "configs[4] (the layers around the attention module are torch stand-ins), one GPU")
    ap.add_argument("--module", action="store_true",
                    help="side measurement, not the bench line: the TimeSelfAttention module (projections + "
                         "attention + residual + LayerNorm) at BASELINE configs[1] per GPU, tensor-pipe mode")
    args = ap.parse_args()
    if args.module:
        module_measurement(args)
        return
    if args.model_step:
        model_step_measurement(args)
        return
    if args.ring:
        CFG["B"] = args.batch
        ring_measurement(args)
        return
    if args.profile:
        args.steps, args.warmup, args.no_e2e, args.no_cpu_baseline = 1, 1, True, True
    CFG["B"] = args.batch
    if args.impl == "reference":
        reference_arm(args)
        return

    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    import cuda_ltc_b200 as ltc
    from cuda_ltc_b200 import _lib

    W = args.warmup if args.profile else max(3, args.warmup)
    K = args.steps
    B, H, S, D = CFG["B"], CFG["H"], CFG["S"], CFG["D"]
    dev = torch.device("cuda", local_rank)
    g = torch.Generator(device=dev).manual_seed(SEED + rank)
    mk = lambda: (torch.randn((B, H, S, D), generator=g, device=dev) * 0.5).bfloat16()
    q, k, v, do = mk(), mk(), mk(), mk()
    o = torch.empty_like(q)
    lse = torch.empty((B, H, S), dtype=torch.float32, device=dev)
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)

    stream = torch.cuda.Stream(device=dev)
    ctx = ltc.Context(local_rank, stream)
    bwd_tensor = ctx.uses_tensor_pipe(q, k, v, causal=True, backward=True)
    kernels_per_step = 1 + (3 if not bwd_tensor else int(os.environ.get("LTCA_BWD_LAUNCHES", "3")))

    def step():
        ctx.attn_fwd(q, k, v, causal=True, mode=_lib.MODE_BF16, out=o, lse=lse)
        ctx.attn_bwd(q, k, v, o, lse, do, causal=True, mode=_lib.MODE_AUTO, dq=dq, dk=dk, dv=dv)

    def barrier():
        torch.cuda.synchronize(dev)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    with torch.cuda.stream(stream):
        for _ in range(W):
            step()
    barrier()

    sampler = ClockSampler(physical_gpu_index(local_rank))
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(K)]
    sampler.start()
    with torch.cuda.stream(stream):
        for i in range(K):
            ev[i][0].record(stream)
            ctx.attn_fwd(q, k, v, causal=True, mode=_lib.MODE_BF16, out=o, lse=lse)
            ev[i][1].record(stream)
            ctx.attn_bwd(q, k, v, o, lse, do, causal=True, mode=_lib.MODE_AUTO, dq=dq, dk=dk, dv=dv)
            ev[i][2].record(stream)
    barrier()
    clocks = sampler.stop()
    total_ms = ev[0][0].elapsed_time(ev[-1][2])
    fwd_ms = sum(e[0].elapsed_time(e[1]) for e in ev) / K
    bwd_ms = sum(e[1].elapsed_time(e[2]) for e in ev) / K
    status = ctx.device_status()

    # ---- per-kernel durations of the backward (events recorded inside the library on the same stream) --
    kern_ms = None
    if bwd_tensor:
        ctx.enable_kernel_timing(True)
        acc = [0.0, 0.0, 0.0]
        Kk = max(3, min(K, 10))
        with torch.cuda.stream(stream):
            for _ in range(Kk):
                ctx.attn_fwd(q, k, v, causal=True, mode=_lib.MODE_BF16, out=o, lse=lse)
                ctx.attn_bwd(q, k, v, o, lse, do, causal=True, mode=_lib.MODE_AUTO, dq=dq, dk=dk, dv=dv)
                for i, x in enumerate(ctx.last_bwd_kernel_ms()):
                    acc[i] += x
        ctx.enable_kernel_timing(False)
        kern_ms = [x / Kk for x in acc]
        barrier()

    # ---- end to end: host buffers in, results back, through the same public call ---------------
    e2e = None
    if not args.no_e2e:
        hq, hk, hv, hdo = (t.cpu().pin_memory() for t in (q, k, v, do))
        ho, hdq, hdk, hdv = (torch.empty_like(t).pin_memory() for t in (hq, hq, hk, hv))
        Ke = max(8, min(K, 20))

        # the library's host-buffer front end: copy in / compute / copy out on three streams, two sets of
        # device buffers, so neighbouring steps overlap; every step still brings its operands from the host
        # and returns its results there inside the timed region
        from cuda_ltc_b200 import HostStepPipeline
        pipe = HostStepPipeline(ctx, stream, q, k, causal=True)
        host_in, host_out = (hq, hk, hv, hdo), (ho, hdq, hdk, hdv)
        pipe.run(host_in, host_out, 2)
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(pipe.s_in)
        pipe.run(host_in, host_out, Ke)
        e1.record(pipe.s_out)
        barrier()
        e2e_ms = e0.elapsed_time(e1) / Ke
        nbytes = q.numel() * 2
        e2e = (e2e_ms, 4 * nbytes, 4 * nbytes)

    # ---- max over ranks --------------------------------------------------------------------------
    from cuda_ltc_b200.shard import reduce_max
    red = reduce_max([total_ms, fwd_ms, bwd_ms, e2e[0] if e2e else 0.0, float(status)] + (kern_ms or []))
    total_ms, fwd_ms, bwd_ms, e2e_ms, status = red[:5]
    if kern_ms:
        kern_ms = red[5:8]

    if rank == 0:
        f_fwd = flops_fwd(B, H, S, D)
        f_step = 3.5 * f_fwd
        ms_per_step = total_ms / K
        value = world * f_step / (ms_per_step * 1e-3) / 1e12
        peaks, peak_kind = measured_peaks()
        peak = peaks.get("bf16_tflops_sustained") or peaks.get("bf16_tflops")
        # Algorithmic FLOPs per launch: one contraction over the causal half is f_fwd / 2.  Forward =
        # 2 contractions; the dK/dV kernel is charged S^T, dP^T, dV, dK (4), the dQ kernel only dQ (1; its
        # own S and dP are recomputation): together the 2.5 x forward of the backward pass.
        kernels = {"attn_fwd4p_sm100_kernel": {"ms": fwd_ms, "flops": f_fwd}}
        if kern_ms:
            kernels["attn_bwd_stats_kernel"] = {"ms": kern_ms[0], "flops": 0.0}
            kernels["attn_bwd_dq4_sm100_kernel"] = {"ms": kern_ms[1], "flops": 0.5 * f_fwd}
            kernels["attn_bwd_dkv4_sm100_kernel"] = {"ms": kern_ms[2], "flops": 2.0 * f_fwd}
        else:
            kernels["attention backward (fp32 path)"] = {"ms": bwd_ms, "flops": 2.5 * f_fwd}
        dom = max(kernels, key=lambda n: kernels[n]["ms"])
        achieved = kernels[dom]["flops"] / (kernels[dom]["ms"] * 1e-3) / 1e12
        # DRAM bytes per launch of that kernel: ncu capture at B=2 (profiles/attention_core_b2_s4096_ncu_full.md),
        # which grows in proportion to batch x heads; None for a kernel that was not captured
        dram_per_bh = {"attn_fwd4p_sm100_kernel": 1.649e6, "attn_bwd_dq4_sm100_kernel": 2.258e6,
                       "attn_bwd_dkv4_sm100_kernel": 2.358e6}
        traffic = dram_per_bh[dom] * B * H if dom in dram_per_bh else None
        line = {
            "metric": "attention fwd+bwd TFLOP/s", "value": value, "unit": "TFLOP/s",
            "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic", "config": workload_config(world),
            "fwd": {"ms": fwd_ms, "tflops_per_gpu": f_fwd / (fwd_ms * 1e-3) / 1e12},
            "bwd": {"ms": bwd_ms, "tflops_per_gpu": 2.5 * f_fwd / (bwd_ms * 1e-3) / 1e12,
                    "tensor_pipe": bool(bwd_tensor)},
            "kernels_ms": {n: round(kernels[n]["ms"], 4) for n in kernels},
            "roofline": {"bound": "tensor", "kernel": dom, "achieved": achieved, "peak": peak,
                         "unit": "TFLOP/s", "frac": achieved / peak,
                         "peak_source": f"{peak_kind} bf16_tflops_sustained", "traffic": traffic,
                         "traffic_unit": "DRAM bytes per launch (ncu, scaled from B=2)",
                         "whole_step_frac": value / world / peak},
            "gpu_launches": kernels_per_step * K,
            "clocks": clocks, "device_status": int(status),
        }
        if e2e:
            line["e2e"] = {"value": world * f_step / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s",
                           "ms_per_step": e2e_ms, "h2d_bytes_per_step": e2e[1], "d2h_bytes_per_step": e2e[2],
                           "how": "HostStepPipeline: copy in / compute / copy out on three streams, two device buffer sets; "
                                  "fill and drain of the pipeline are inside the timed region"}
        if world == 1 and not args.no_cpu_baseline:
            cores = os.cpu_count() or 1
            n_bh = max(8, min(cores, 64))
            tf, dt, threads = run_cpu_sample(n_bh)
            line["cpu_baseline"] = {"value": tf, "unit": "TFLOP/s", "cores": threads, "kind": "port",
                                    "sample": f"{n_bh} of {B * H} (batch, head) pairs, forward + backward, "
                                              f"fp64, {dt:.1f} s"}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
