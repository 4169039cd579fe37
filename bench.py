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
        """One NVML query pair every 2 ms (the timed region of the default run is about 33 ms)."""
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
            self._stop.wait(0.002)

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
                "reasons": sorted(self.reasons), "samples": len(s)}


def pin_to_gpu_numa_node(torch, local_rank: int) -> dict:
    """Moves this process onto the CPUs of the NUMA node its GPU hangs off, so that the pinned host buffers
    allocated afterwards (first touch) and the copy threads sit beside the GPU's PCIe root.  Returns what was
    found; does nothing where the node is not exposed (numa_node = -1, as inside most virtual machines)."""
    info = {"numa_node": None, "applied": False}
    try:
        pr = torch.cuda.get_device_properties(local_rank)
        bdf = f"{pr.pci_domain_id:04x}:{pr.pci_bus_id:02x}:{pr.pci_device_id:02x}.0"
        info["pci"] = bdf
        with open(f"/sys/bus/pci/devices/{bdf}/numa_node") as f:
            node = int(f.read().strip())
        info["numa_node"] = node
        if node < 0:
            return info
        with open(f"/sys/devices/system/node/node{node}/cpulist") as f:
            cpus = set()
            for part in f.read().strip().split(","):
                a, _, b = part.partition("-")
                cpus.update(range(int(a), int(b or a) + 1))
        allowed = os.sched_getaffinity(0) & cpus
        if allowed:
            os.sched_setaffinity(0, allowed)
            info["applied"], info["cpus"] = True, len(allowed)
    except Exception as e:
        info["error"] = repr(e)[:120]
    return info


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


def reference_cuda_module_timings():
    """The reference's own CUDA build timed on this GPU: its cuDNN TimeSelfAttention (forward, backwardWeights,
    backward as its model calls them) beside this library's C++ binding in the same process, at the two module
    shapes of the benchmark configurations.  The binary is oracle/_ref/shim_driver, built in advance from the
    reference checkout (oracle/Makefile); absent binary, absent GPU or a cuDNN refusal are recorded as text."""
    import subprocess
    exe = os.path.join(ROOT, "oracle", "_ref", "shim_driver")
    if not os.path.exists(exe):
        return {"unavailable": "oracle/_ref/shim_driver not built (needs the reference checkout)"}
    out = {}
    for name, shape, iters in (("config2_B32_S256_E512_H8", (32, 256, 512, 8), 10),
                               ("config5_B64_S512_E512_H8", (64, 512, 512, 8), 5)):
        try:
            r = subprocess.run([exe, "time", *map(str, shape), str(iters)], capture_output=True, text=True,
                               timeout=240)
            lines = [ln for ln in r.stdout.splitlines() if ln.startswith("{")]
            out[name] = json.loads(lines[-1]) if lines else {
                "unavailable": (r.stderr.strip() or r.stdout.strip() or f"exit code {r.returncode}")[-300:]}
        except Exception as e:      # time-out, unreadable output
            out[name] = {"unavailable": repr(e)[:300]}
    return out


def reference_arm(args):
    """CPU arm: the reference has no CPU implementation of this path (all of it is CUDA and its
    own kernels cannot run this configuration), so the timed code is the repository's fp64
    OpenMP port of the same arithmetic, on all host threads, on a bounded sample per step.  The line also
    carries `reference_cuda`: the reference's own cuDNN module timed on the GPU (other shapes, other
    semantics: per-head width = model width, no causal mask), for the module-level configurations."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    import oracle
    oracle.set_num_threads(cores)           # a launcher may have exported OMP_NUM_THREADS=1
    n_bh = max(8, min(cores, 64))
    for _ in range(args.warmup if args.warmup < 2 else 1):
        run_cpu_sample(max(2, n_bh // 4), cores)
    t_total, fl_total = 0.0, 0.0
    threads = 1
    for _ in range(args.steps):
        tf, dt, threads = run_cpu_sample(n_bh, cores)
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
    if not args.no_reference_cuda:
        line["reference_cuda"] = reference_cuda_module_timings()
    print(json.dumps(line), flush=True)


def workload_config(n_gpus):
    return {"workload": f"attention core fwd+bwd, B={CFG['B']} H=16 S=4096 D=64 causal, bf16 storage / fp32 "
                        "accumulate (BASELINE configs[2]" + ("" if CFG["B"] == 8 else ", reduced batch") + "); per GPU",
            "global_batch": CFG["B"] * n_gpus, "heads": CFG["H"], "seq_len": CFG["S"], "head_dim": CFG["D"],
            "parallelism": f"batch x head partition over {n_gpus} GPU(s), no collective",
            "l2": f"inputs ({32 * CFG['B']} MB per step) exceed the 126 MB L2; no explicit flush"}


def _timed(torch, f, n=20, w=3, flush=None):
    """Mean per-call milliseconds from one CUDA-event pair per call, all calls enqueued before a single
    synchronize (the flush kernel or the previous call keeps the GPU busy while the host prepares the next
    launch, so host overhead stays outside the event pairs).  `flush`: a buffer larger than L2 that is
    rewritten before every call, for inputs that would otherwise stay in L2."""
    for _ in range(w):
        f()
    torch.cuda.synchronize()
    evs = []
    for _ in range(n):
        if flush is not None:
            flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        f()
        e1.record()
        evs.append((e0, e1))
    torch.cuda.synchronize()
    return sum(a.elapsed_time(b) for a, b in evs) / n


def other_configs(torch, ctx, peaks):
    """The other BASELINE configurations on one GPU (side record of the bench line, not the metric):
    config 1 (FlashAttention forward, fp32, B2 H4 S64 D32), config 2 (TimeSelfAttention B32 S256 E512 H8 causal:
    attention core and whole module, forward and backward), config 4 (decode step, HBM bound) and config 5's
    attention core (B64 H8 S512 D64 causal).  Small inputs are timed with an L2 flush before every call."""
    import numpy as np
    from cuda_ltc_b200 import _lib
    out = {}
    dev = torch.device("cuda", ctx.device)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    g = torch.Generator(device=dev).manual_seed(SEED + 7)
    rn = lambda *shape: torch.randn(shape, generator=g, device=dev)
    # config 1
    q, k, v = rn(2, 4, 64, 32), rn(2, 4, 64, 32), rn(2, 4, 64, 32)
    ms = _timed(torch, lambda: ctx.attn_fwd(q, k, v, mode=_lib.MODE_AUTO), flush=flush)
    ms_split = _timed(torch, lambda: ctx.attn_fwd(q, k, v, mode=_lib.MODE_SPLIT), flush=flush)
    out["config1_fa_fwd_fp32_B2_H4_S64_D32"] = {
        "fwd_us": ms * 1e3, "bound": "launch latency (4.2 MFLOP, 256 KiB)",
        "tensor_pipe": ctx.uses_tensor_pipe(q, k, v),
        "split_precision_tensor_pipe_fwd_us": ms_split * 1e3}
    # config 2: attention core
    fl2 = flops_fwd(32, 8, 256, 64)
    q, k, v, do = (rn(32, 8, 256, 64) for _ in range(4))
    core = {}
    for name, mode, conv in (("fp32_storage_tensor_pipe", _lib.MODE_BF16, lambda t: t),
                             ("bf16_storage_tensor_pipe", _lib.MODE_BF16, lambda t: t.bfloat16()),
                             ("fp32_storage_split_precision_tensor_pipe", _lib.MODE_SPLIT, lambda t: t),
                             ("fp32_storage_exact", _lib.MODE_FP32, lambda t: t)):
        qq, kk, vv, dd = (conv(t) for t in (q, k, v, do))
        o, lse = ctx.attn_fwd(qq, kk, vv, causal=True, mode=mode)
        f_ms = _timed(torch, lambda: ctx.attn_fwd(qq, kk, vv, causal=True, mode=mode, out=o, lse=lse), flush=flush)
        b_ms = _timed(torch, lambda: ctx.attn_bwd(qq, kk, vv, o, lse, dd, causal=True, mode=mode), flush=flush)
        core[name] = {"fwd_us": f_ms * 1e3, "bwd_us": b_ms * 1e3, "fwd_tflops": fl2 / f_ms / 1e9,
                      "fwdbwd_tflops": 3.5 * fl2 / (f_ms + b_ms) / 1e9}
    out["config2_core_B32_H8_S256_D64_causal"] = core
    # config 2: the whole module (projections + core + residual + LayerNorm)
    B, S, E, H, W = 32, 256, 512, 8, 64
    x, dy = rn(B * S, E), rn(B * S, E)
    lim = math.sqrt(6.0 / (2 * E))
    ws = [(torch.rand((E, H * W), generator=g, device=dev) * 2 - 1) * lim for _ in range(3)]
    wo = (torch.rand((H * W, E), generator=g, device=dev) * 2 - 1) * lim
    gamma, beta = torch.ones(E, device=dev), torch.zeros(E, device=dev)
    gemm = 2.0 * B * S * E * H * W
    mod = {}
    for name, mode in (("tensor_pipe", _lib.MODE_BF16), ("exact_fp32", _lib.MODE_FP32)):
        kw = dict(scale=1 / math.sqrt(W), causal=True, time_major=False, mode=mode)
        n = 20 if mode == _lib.MODE_BF16 else 5
        f_ms = _timed(torch, lambda: ctx.tsa_fwd(x, *ws, wo, B, S, H, W, gamma=gamma, beta=beta, **kw), n=n, flush=flush)
        b_ms = _timed(torch, lambda: ctx.tsa_bwd(x, *ws, wo, dy, B, S, H, W, **kw), n=n, flush=flush)
        mod[name] = {"fwd_us": f_ms * 1e3, "bwd_incl_recomputed_fwd_us": b_ms * 1e3,
                     "fwd_tflops": (4 * gemm + fl2) / f_ms / 1e9,
                     "bwd_tflops": (8 * gemm + 2.5 * fl2) / b_ms / 1e9}
    out["config2_module_B32_S256_E512_H8_causal"] = mod
    # the same module in the REFERENCE's form (every head as wide as the model, scale 1, no mask, time-major rows:
    # what its cuDNN module computes; `--impl reference` times that module itself under `reference_cuda`)
    Wr = E
    wsr = [(torch.rand((E, H * Wr), generator=g, device=dev) * 2 - 1) * lim for _ in range(3)]
    wor = (torch.rand((H * Wr, E), generator=g, device=dev) * 2 - 1) * lim
    kwr = dict(scale=1.0, causal=False, time_major=True, mode=_lib.MODE_AUTO)
    f_ms = _timed(torch, lambda: ctx.tsa_fwd(x, *wsr, wor, B, S, H, Wr, gamma=gamma, beta=beta, **kwr), n=10, flush=flush)
    b_ms = _timed(torch, lambda: ctx.tsa_bwd(x, *wsr, wor, dy, B, S, H, Wr, **kwr), n=10, flush=flush)
    gemm_r = 2.0 * B * S * E * H * Wr
    core_r = 4.0 * B * H * S * S * Wr
    out["config2_module_reference_form_head_width_512"] = {
        "fwd_us": f_ms * 1e3, "bwd_incl_recomputed_fwd_us": b_ms * 1e3,
        "fwd_tflops": (4 * gemm_r + core_r) / f_ms / 1e9,
        "path": "written-out scores, batched tcgen05 GEMMs, two-term Q/K operands"}
    del wsr, wor
    # config 5: attention core
    fl5 = flops_fwd(64, 8, 512, 64)
    q, k, v, do = (rn(64, 8, 512, 64).bfloat16() for _ in range(4))
    o, lse = ctx.attn_fwd(q, k, v, causal=True, mode=_lib.MODE_BF16)
    f_ms = _timed(torch, lambda: ctx.attn_fwd(q, k, v, causal=True, mode=_lib.MODE_BF16, out=o, lse=lse), flush=flush)
    b_ms = _timed(torch, lambda: ctx.attn_bwd(q, k, v, o, lse, do, causal=True, mode=_lib.MODE_BF16), flush=flush)
    out["config5_core_B64_H8_S512_D64_causal_bf16"] = {
        "fwd_us": f_ms * 1e3, "bwd_us": b_ms * 1e3, "fwd_tflops": fl5 / f_ms / 1e9,
        "fwdbwd_tflops": 3.5 * fl5 / (f_ms + b_ms) / 1e9}
    del q, k, v, do, o, lse
    # config 4: decode step, HBM bound.  K/V cache = 1 GB > L2; algorithmic bytes = keys and values actually
    # visible (sum of kv_len x H x D x 4 B x 2) + q and o (2 x B x H x D x 4 B) + the lengths (4 B).
    B, H, S, D = 256, 8, 1024, 64
    qd, kd, vd = rn(B, H, 1, D), rn(B, H, S, D), rn(B, H, S, D)
    L = torch.from_numpy(np.random.default_rng(10).integers(1, S + 1, size=B).astype(np.int32)).to(dev)
    od, lsed = ctx.attn_decode(qd, kd, vd, kv_len=L)
    dec = {}
    for name, lens in (("kv_len_uniform_1_to_1024", L),
                       ("kv_len_all_1024", torch.full((B,), S, dtype=torch.int32, device=dev))):
        nbytes = int(lens.sum().item()) * H * D * 4 * 2 + 2 * B * H * D * 4 + 4 * B
        ms = _timed(torch, lambda: ctx.attn_decode(qd, kd, vd, kv_len=lens, out=od, lse=lsed), n=50, flush=flush)
        ms_b2b = _timed(torch, lambda: ctx.attn_decode(qd, kd, vd, kv_len=lens, out=od, lse=lsed), n=50)
        dec[name] = {"us": ms * 1e3, "algorithmic_bytes": nbytes, "achieved_gbs": nbytes / ms / 1e6,
                     "frac_of_hbm_peak": nbytes / ms / 1e6 / peaks["hbm_gbs"],
                     "back_to_back_us": ms_b2b * 1e3, "back_to_back_gbs": nbytes / ms_b2b / 1e6,
                     "back_to_back_frac_of_hbm_peak": nbytes / ms_b2b / 1e6 / peaks["hbm_gbs"]}
    dec["bound"] = "hbm"
    dec["peak_gbs"] = peaks["hbm_gbs"]
    dec["note"] = ("us / achieved_gbs: a 256 MB buffer is zeroed before every launch (L2 flushed, and the launch "
                   "starts behind the flush's write-back); back_to_back_*: launches in a row, the cache (1 GB) "
                   "exceeds L2 in any case")
    out["config4_decode_B256_H8_S1024_D64_fp32"] = dec
    return out


def dram_bytes_record():
    """DRAM bytes per (batch, head) pair of the three main kernels, from the ncu capture summarised beside the
    file (profiles/attention_core_dram_bytes.json carries the commit the capture was taken at)."""
    try:
        with open(os.path.join(ROOT, "profiles", "attention_core_dram_bytes.json")) as f:
            return json.load(f)
    except Exception:
        return None


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
    if args.reference_form:
        W = E                                           # the reference's module: every head as wide as the model
    g = torch.Generator(device="cuda").manual_seed(SEED + rank)
    x = torch.randn((B * S, E), generator=g, device="cuda")
    dy = torch.randn((B * S, E), generator=g, device="cuda")
    gw = torch.Generator(device="cuda").manual_seed(SEED)
    lim = math.sqrt(6.0 / (2 * E))
    ws = [(torch.rand((E, H * W), generator=gw, device="cuda") * 2 - 1) * lim for _ in range(3)]
    wo = (torch.rand((H * W, E), generator=gw, device="cuda") * 2 - 1) * lim
    gamma, beta = torch.ones(E, device="cuda"), torch.zeros(E, device="cuda")
    kw = dict(scale=1 / math.sqrt(W), causal=True, time_major=False, mode=_lib.MODE_BF16)
    if args.reference_form:
        kw = dict(scale=1.0, causal=False, time_major=True, mode=_lib.MODE_AUTO)
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
    core = 4.0 * B * world * H * S * S * W / (1 if args.reference_form else 2)
    print(json.dumps({"workload": f"TimeSelfAttention module, B=32 per GPU, S=256 E=512 H=8 W={W} "
                                  + ("scale 1 unmasked (reference form), AUTO mode" if args.reference_form else
                                     "causal, tensor-pipe mode") + "; weight gradients summed over the ranks",
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
    from cuda_ltc_b200 import gather, ring
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
    gathered = bool(args.gather)
    # (with gathered K/V the collectives do not run beside the kernels: no SMs are set aside for them)
    ops = ring.CudaOps(ctx, comm_sms=0 if gathered else args.comm_sms)
    cache = {}                                          # scratch and receive buffers live across the steps
    n, w = max(5, args.steps), max(3, args.warmup)

    def step():
        if gathered:
            o, lse, kf, vf = gather.gathered_attention_fwd(ops, q, k, v, rank, world, causal=True, cache=cache)
            gather.gathered_attention_bwd(ops, q, kf, vf, o, lse, do, rank, world, causal=True, cache=cache,
                                          reduce_in_bf16=bool(args.reduce_bf16))
            return
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
    if gathered:
        print(json.dumps({"workload": f"attention fwd+bwd, B={B} H={H} S={S} D={D} causal bf16, sequence dealt out "
                                      f"over {world} GPU(s), K/V gathered, dK/dV reduce-scattered (strong scaling)",
                          "n_gpus": world, "ms_per_step": ms, "tflops_whole_job": flops / ms / 1e9,
                          "all_gather_bytes_received_per_gpu": 2 * B * H * (S - L) * D * 2,
                          "reduce_scatter_bytes_sent_per_gpu": 2 * B * H * (S - L) * D * (2 if args.reduce_bf16 else 4),
                          "device_status": status}))
        return
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
    ap.add_argument("--no-sustained", action="store_true", help="skip the two-second repetition of the step")
    ap.add_argument("--no-configs", action="store_true", help="skip the side record of the other configurations")
    ap.add_argument("--no-reference-cuda", action="store_true",
                    help="--impl reference: skip the GPU timing of the reference's cuDNN module")
    ap.add_argument("--batch", type=int, default=CFG["B"],
                    help="sequences per GPU; anything but the default is a reduced case for profiler captures")
    ap.add_argument("--profile", action="store_true",
                    help="profiler capture mode: 1 warm-up, 1 step, no end-to-end or CPU legs (not a bench value)")
    ap.add_argument("--seq-len", type=int, default=0, help="sequence length of the --ring measurement (default: the "
                                                           "bench configuration's)")
    ap.add_argument("--comm-sms", type=int, default=16,
                    help="--ring: SMs the attention kernels leave free for the exchange's copy kernels")
    ap.add_argument("--reduce-bf16", action="store_true",
                    help="with --gather: the shares of dK / dV travel and are summed as bf16 instead of fp32")
    ap.add_argument("--gather", action="store_true",
                    help="with --ring's workload: gather K/V and reduce-scatter dK/dV instead of the ring exchange")
    ap.add_argument("--ring", action="store_true",
                    help="side measurement, not the bench line: the same problem with the sequence dealt out over "
                         "the ranks and K/V exchanged round a ring (launch one rank per GPU)")
    ap.add_argument("--model-step", action="store_true",
                    help="side measurement, not the bench line: attention's share of a step shaped like BASELINE "
                         "configs[4] (the layers around the attention module are torch stand-ins), one GPU")
    ap.add_argument("--reference-form", action="store_true",
                    help="with --module: head width = E, scale 1, no mask, time-major rows (the reference's module)")
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
    if args.ring or args.gather:
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

    numa = pin_to_gpu_numa_node(torch, local_rank) if not args.no_e2e else None
    stream = torch.cuda.Stream(device=dev)
    ctx = ltc.Context(local_rank, stream)
    bwd_tensor = ctx.uses_tensor_pipe(q, k, v, causal=True, backward=True)
    kernels_per_step = 1 + 3        # forward; backward = row statistics + fused kernel + dQ conversion (fp32 path: 3 too)

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

    # ---- the bit-reproducible backward (two kernels, seven contractions), for comparison --------------------
    det_bwd_ms = None
    if bwd_tensor and not args.profile and not args.no_configs:
        with torch.cuda.stream(stream):
            ctx.attn_bwd(q, k, v, o, lse, do, causal=True, mode=_lib.MODE_AUTO, dq=dq, dk=dk, dv=dv, deterministic=True)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(5):
                ctx.attn_bwd(q, k, v, o, lse, do, causal=True, mode=_lib.MODE_AUTO, dq=dq, dk=dk, dv=dv,
                             deterministic=True)
            e1.record(stream)
        barrier()
        det_bwd_ms = e0.elapsed_time(e1) / 5

    # ---- the same step repeated for about two seconds: the figure under the power cap --------------------
    sustained = None
    if world == 1 and not args.profile and not args.no_sustained:
        n_sus = max(K, int(math.ceil(2000.0 / max(total_ms / K, 1e-3))))
        sampler2 = ClockSampler(physical_gpu_index(local_rank))
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        sampler2.start()
        with torch.cuda.stream(stream):
            e0.record(stream)
            for _ in range(n_sus):
                step()
            e1.record(stream)
        barrier()
        sustained = (e0.elapsed_time(e1) / n_sus, n_sus, sampler2.stop())

    # ---- strong scaling: the SAME global problem (B x H pairs of one rank's batch) dealt out over the ranks --
    strong_ms = None
    if world > 1 and not args.profile:
        from cuda_ltc_b200.shard import unit_range
        r = unit_range(B * H, world, rank)
        sl = lambda t: t.reshape(1, B * H, S, -1)[:, r.start:r.stop]
        sq, sk, sv, sdo, so, sdq, sdk, sdv = (sl(t) for t in (q, k, v, do, o, dq, dk, dv))
        slse = lse.reshape(1, B * H, S)[:, r.start:r.stop]

        def strong_step():
            ctx.attn_fwd(sq, sk, sv, causal=True, mode=_lib.MODE_BF16, out=so, lse=slse)
            ctx.attn_bwd(sq, sk, sv, so, slse, sdo, causal=True, mode=_lib.MODE_AUTO, dq=sdq, dk=sdk, dv=sdv)

        with torch.cuda.stream(stream):
            for _ in range(W):
                strong_step()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(stream):
            e0.record(stream)
            for _ in range(K):
                strong_step()
            e1.record(stream)
        barrier()
        strong_ms = e0.elapsed_time(e1) / K

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
        # the same pipeline with the kernels left out: what the host link alone allows on this box
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(pipe.s_in)
        pipe.run(host_in, host_out, Ke, compute=False)
        e1.record(pipe.s_out)
        barrier()
        copy_ms = e0.elapsed_time(e1) / Ke
        e2e = (e2e_ms, 4 * nbytes, 4 * nbytes, copy_ms)

    # ---- max over ranks --------------------------------------------------------------------------
    from cuda_ltc_b200.shard import reduce_max
    red = reduce_max([total_ms, fwd_ms, bwd_ms, e2e[0] if e2e else 0.0, float(status),
                      e2e[3] if e2e else 0.0, strong_ms or 0.0] + (kern_ms or []))
    total_ms, fwd_ms, bwd_ms, e2e_ms, status, copy_ms, strong_ms = red[:7]
    if kern_ms:
        kern_ms = red[7:10]

    if rank == 0:
        f_fwd = flops_fwd(B, H, S, D)
        f_step = 3.5 * f_fwd
        ms_per_step = total_ms / K
        value = world * f_step / (ms_per_step * 1e-3) / 1e12
        peaks, peak_kind = measured_peaks()
        # the timed region is tens of milliseconds at full clock: the comparator is the BURST GEMM figure; the
        # sustained figure is used only for the two-second leg below
        peak = peaks.get("bf16_tflops") or peaks.get("bf16_tflops_sustained")
        # Algorithmic FLOPs per launch: one contraction over the causal half is f_fwd / 2.  Forward =
        # 2 contractions; the dK/dV kernel is charged S^T, dP^T, dV, dK (4), the dQ kernel only dQ (1; its
        # own S and dP are recomputation): together the 2.5 x forward of the backward pass.
        kernels = {"attn_fwd4p_sm100_kernel": {"ms": fwd_ms, "flops": f_fwd}}
        if kern_ms:
            # bf16 storage takes the fused backward: row statistics (which also clear the fp32 dQ accumulator),
            # one kernel with the five contractions (2.5 x forward), and the conversion of the accumulator
            kernels["attn_bwd_stats_kernel"] = {"ms": kern_ms[0], "flops": 0.0}
            kernels["attn_bwd_fused_sm100_kernel"] = {"ms": kern_ms[1], "flops": 2.5 * f_fwd}
            kernels["attn_bwd_dq_convert_kernel"] = {"ms": kern_ms[2], "flops": 0.0}
        else:
            kernels["attention backward (fp32 path)"] = {"ms": bwd_ms, "flops": 2.5 * f_fwd}
        dom = max(kernels, key=lambda n: kernels[n]["ms"])
        achieved = kernels[dom]["flops"] / (kernels[dom]["ms"] * 1e-3) / 1e12
        # DRAM bytes per launch of that kernel: an ncu capture at B=2 scaled by batch x heads (traffic grows in
        # proportion); None for a kernel without a capture
        dram = dram_bytes_record()
        per_bh = (dram or {}).get("dram_bytes_per_batch_head", {}).get(dom)
        traffic = per_bh * B * H if per_bh else None
        line = {
            "metric": "attention fwd+bwd TFLOP/s", "value": value, "unit": "TFLOP/s",
            "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic", "config": workload_config(world),
            "fwd": {"ms": fwd_ms, "tflops_per_gpu": f_fwd / (fwd_ms * 1e-3) / 1e12},
            "bwd": {"ms": bwd_ms, "tflops_per_gpu": 2.5 * f_fwd / (bwd_ms * 1e-3) / 1e12,
                    "tensor_pipe": bool(bwd_tensor), "bit_reproducible_variant_ms": det_bwd_ms},
            "kernels_ms": {n: round(kernels[n]["ms"], 4) for n in kernels},
            "roofline": {"bound": "tensor", "kernel": dom, "achieved": achieved, "peak": peak,
                         "unit": "TFLOP/s", "frac": achieved / peak,
                         "peak_source": f"{peak_kind} bf16_tflops (burst: the timed region is short)",
                         "traffic": traffic,
                         "traffic_source": (f"ncu capture at B=2 scaled by batch x heads, kernels as of commit "
                                            f"{dram.get('commit')}" if dram and traffic else None),
                         "whole_step_frac": value / world / peak, "fwd_frac": f_fwd / (fwd_ms * 1e-3) / 1e12 / peak},
            "gpu_launches": kernels_per_step * K,
            "clocks": clocks, "device_status": int(status),
        }
        if sustained:
            s_ms, s_n, s_clk = sustained
            s_peak = peaks.get("bf16_tflops_sustained") or peak
            line["sustained"] = {"steps": s_n, "ms_per_step": s_ms, "tflops": f_step / (s_ms * 1e-3) / 1e12,
                                 "frac_of_sustained_peak": f_step / (s_ms * 1e-3) / 1e12 / s_peak,
                                 "peak": s_peak, "peak_source": f"{peak_kind} bf16_tflops_sustained",
                                 "clocks": s_clk}
        if strong_ms:
            line["strong"] = {"workload": f"the same global B={B} x H={H} pairs dealt out over the ranks",
                              "pairs_per_gpu": B * H // world, "ms_per_step": strong_ms,
                              "tflops_whole_job": f_step / (strong_ms * 1e-3) / 1e12,
                              "speedup_vs_one_gpu": ms_per_step / strong_ms}
        if e2e:
            line["e2e"] = {"value": world * f_step / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s",
                           "ms_per_step": e2e_ms, "h2d_bytes_per_step": e2e[1], "d2h_bytes_per_step": e2e[2],
                           "how": "HostStepPipeline: copy in / compute / copy out on three streams, two device buffer sets; "
                                  "fill and drain of the pipeline are inside the timed region",
                           "copy_only": {"ms_per_step": copy_ms,
                                         "gbs_per_gpu_each_direction": e2e[1] / (copy_ms * 1e-3) / 1e9,
                                         "gbs_whole_box_both_directions": world * (e2e[1] + e2e[2]) / (copy_ms * 1e-3) / 1e9,
                                         "note": "the same pipeline without the kernels: the host link's share"},
                           "numa": numa}
        if world == 1 and not args.no_cpu_baseline:
            cores = os.cpu_count() or 1
            n_bh = max(8, min(cores, 64))
            tf, dt, threads = run_cpu_sample(n_bh, cores)
            line["cpu_baseline"] = {"value": tf, "unit": "TFLOP/s", "cores": threads, "kind": "port",
                                    "sample": f"{n_bh} of {B * H} (batch, head) pairs, forward + backward, "
                                              f"fp64, {dt:.1f} s"}
        if world == 1 and not args.profile and not args.no_configs:
            try:
                with torch.cuda.stream(stream):         # the context's stream: the event pairs must sit on it
                    line["configs"] = other_configs(torch, ctx, peaks)
                line["configs"]["device_status"] = ctx.device_status()
            except Exception as e:          # a side record must not cost the bench line
                line["configs"] = {"unavailable": repr(e)[:300]}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
