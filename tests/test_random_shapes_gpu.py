"""Randomised shapes, masks and flags through every GPU path against the fp64 oracle: ragged sizes, more queries
than keys, key lengths, dense masks, clamps, every head width and mode, the module with and without its kept
forward and kept weight copies.  Fixed seeds; every case also checks the device status word (a bounded wait that ran
out would show there)."""
import math

import numpy as np
import pytest

import oracle
from util import bf16_round, rel_l2

pytestmark = pytest.mark.gpu


def _dev(a, dtype=None):
    import torch
    if a is None:
        return None
    t = torch.from_numpy(np.ascontiguousarray(a)).cuda()
    return t if dtype is None else t.to(dtype)


def test_streaming_kernels_random_shapes(ctx):
    """Head width 64, bf16 storage: forward, the fused backward and the two-kernel backward."""
    import torch
    from cuda_ltc_b200 import _lib
    rng = np.random.default_rng(101)
    done = 0
    while done < 60:
        B, H = int(rng.integers(1, 4)), int(rng.integers(1, 5))
        Sq, Sk = int(rng.integers(1, 1800)), int(rng.integers(1, 1800))
        if B * H * Sq * Sk > 4e6:
            continue
        causal = bool(rng.integers(0, 2))
        L = rng.integers(1, Sk + 1, size=B).astype(np.int32) if rng.random() < 0.3 else None
        q, k, v, do = (bf16_round((rng.standard_normal((B, H, S, 64)) * 0.5).astype(np.float32))
                       for S in (Sq, Sk, Sk, Sq))
        o_ref, _ = oracle.attn_fwd(q, k, v, 0.125, causal, None, L, 0.0)
        ref = oracle.attn_bwd(q, k, v, do, 0.125, causal, None, L, 0.0)
        tq, tk, tv, tdo = (_dev(a, torch.bfloat16) for a in (q, k, v, do))
        kw = dict(scale=0.125, causal=causal, kv_len=_dev(L), mode=_lib.MODE_BF16)
        o, lse = ctx.attn_fwd(tq, tk, tv, **kw)
        what = (B, H, Sq, Sk, causal, L is not None)
        assert np.abs(o.float().cpu().numpy() - o_ref).max() < 1.2e-2, what
        for det in (False, True):
            grads = ctx.attn_bwd(tq, tk, tv, o, lse, tdo, deterministic=det, **kw)
            torch.cuda.synchronize()
            assert ctx.device_status() == 0, what
            for g, r in zip(grads, ref):
                assert np.abs(g.float().cpu().numpy() - r).max() <= 1.2e-2 * max(1.0, np.abs(r).max()), (what, det)
        done += 1


def test_streaming_kernels_random_shapes_many_pairs(ctx):
    """The same with enough (batch, head) pairs that the persistent kernels hold more work items than there are SMs
    and every CTA walks through several of them, many without work: short key lengths in most batch entries, more
    queries than keys under the causal mask.  bf16 or fp32 storage."""
    import torch
    from cuda_ltc_b200 import _lib
    rng = np.random.default_rng(404)
    done = 0
    while done < 14:
        B, H = int(rng.integers(2, 6)), int(rng.integers(8, 17))
        Sq, Sk = int(rng.integers(300, 1300)), int(rng.integers(300, 1300))
        if B * H * Sq * Sk > 6e7:
            continue
        causal = bool(rng.integers(0, 2))
        L = None
        if rng.random() < 0.7:
            L = np.where(rng.random(B) < 0.7, rng.integers(1, 130, size=B), rng.integers(1, Sk + 1, size=B)).astype(np.int32)
        q, k, v, do = (bf16_round((rng.standard_normal((B, H, S, 64)) * 0.5).astype(np.float32))
                       for S in (Sq, Sk, Sk, Sq))
        o_ref, _ = oracle.attn_fwd(q, k, v, 0.125, causal, None, L, 0.0)
        ref = oracle.attn_bwd(q, k, v, do, 0.125, causal, None, L, 0.0)
        dt = torch.float32 if rng.random() < 0.35 else torch.bfloat16
        tq, tk, tv, tdo = (_dev(a, dt) for a in (q, k, v, do))
        kw = dict(scale=0.125, causal=causal, kv_len=_dev(L), mode=_lib.MODE_BF16)
        o, lse = ctx.attn_fwd(tq, tk, tv, **kw)
        what = (B, H, Sq, Sk, causal, None if L is None else L.tolist(), str(dt))
        assert np.abs(o.float().cpu().numpy() - o_ref).max() < 1.2e-2, what
        for det in (False, True):
            grads = ctx.attn_bwd(tq, tk, tv, o, lse, tdo, deterministic=det, **kw)
            torch.cuda.synchronize()
            assert ctx.device_status() == 0, what
            for g, r in zip(grads, ref):
                assert np.abs(g.float().cpu().numpy() - r).max() <= 1.2e-2 * max(1.0, np.abs(r).max()), (what, det)
        done += 1


def test_written_out_scores_random_shapes(ctx):
    """Every head width that is a multiple of 8, fp32 storage, the bf16 and the split-precision mode, all mask
    kinds and a clamp.  The bf16 mode is compared on bf16-rounded inputs (with a clamp, a score at the threshold
    may otherwise fall on the other side of it)."""
    import torch
    from cuda_ltc_b200 import _lib
    rng = np.random.default_rng(202)
    done = 0
    while done < 120:
        B, H = int(rng.integers(1, 4)), int(rng.integers(1, 4))
        D = int(rng.choice([8, 16, 24, 32, 40, 64, 128, 256]))
        Sq, Sk = int(rng.integers(1, 400)), int(rng.integers(1, 400))
        causal = bool(rng.integers(0, 2))
        clamp = 4.0 if rng.random() < 0.3 else 0.0
        split = rng.random() < 0.5
        if not split and D == 64:
            continue                                        # that width belongs to the streaming kernels
        q, k, v, do = (rng.standard_normal((B, H, S, D)).astype(np.float32) for S in (Sq, Sk, Sk, Sq))
        if not split:
            q, k, v, do = (bf16_round(a) for a in (q, k, v, do))
        L = rng.integers(1, Sk + 1, size=B).astype(np.int32) if rng.random() < 0.3 else None
        m = (rng.random((B, Sq, Sk)) < 0.8).astype(np.float32) if rng.random() < 0.3 else None
        sc = 1.0 / math.sqrt(D)
        o_ref, _ = oracle.attn_fwd(q, k, v, sc, causal, m, L, clamp)
        ref = oracle.attn_bwd(q, k, v, do, sc, causal, m, L, clamp)
        tq, tk, tv, tdo = (_dev(a) for a in (q, k, v, do))
        kw = dict(scale=sc, causal=causal, kv_len=_dev(L), keep_mask=_dev(m), score_clamp=clamp,
                  mode=_lib.MODE_SPLIT if split else _lib.MODE_BF16)
        o, lse = ctx.attn_fwd(tq, tk, tv, **kw)
        grads = ctx.attn_bwd(tq, tk, tv, o, lse, tdo, **kw)
        torch.cuda.synchronize()
        what = (B, H, Sq, Sk, D, causal, clamp, split, L is not None, m is not None)
        assert ctx.device_status() == 0, what
        tol = 2e-4
        assert np.abs(o.cpu().numpy() - o_ref).max() < tol * max(1.0, np.abs(v).max()), what
        for g, r in zip(grads, ref):
            assert np.abs(g.cpu().numpy() - r).max() <= tol * max(1.0, np.abs(r).max()), what
        done += 1


def test_module_random_shapes(ctx):
    """The TimeSelfAttention module in every mode, compact and reference form, with and without biases, the kept
    forward and the kept weight copies."""
    import torch
    from cuda_ltc_b200 import _lib
    rng = np.random.default_rng(303)
    done = 0
    while done < 150:
        E, H = int(rng.choice([32, 64, 128, 256])), int(rng.choice([1, 2, 4]))
        W = E if rng.random() < 0.4 else E // H
        if W % 8:
            continue
        B, S = int(rng.integers(1, 5)), int(rng.integers(2, 90))
        mode = int(rng.choice([_lib.MODE_AUTO, _lib.MODE_BF16, _lib.MODE_FP32]))
        causal, tm, biases = bool(rng.integers(0, 2)), bool(rng.integers(0, 2)), rng.random() < 0.4
        scale = 1.0 if W == E else 1.0 / math.sqrt(W)
        amp = 0.2 if W == E else 1.0
        HW = H * W
        lim = math.sqrt(6.0 / (E + W))
        x = (0.5 * rng.standard_normal((B * S, E))).astype(np.float32)
        dy = rng.standard_normal((B * S, E)).astype(np.float32)
        wq, wk = (rng.uniform(-lim, lim, (E, HW)).astype(np.float32) * amp for _ in range(2))
        wv = rng.uniform(-lim, lim, (E, HW)).astype(np.float32)
        wo = rng.uniform(-lim, lim, (HW, E)).astype(np.float32)
        bq, bk, bv = ((0.1 * rng.standard_normal(HW)).astype(np.float32) if biases else None for _ in range(3))
        gamma, beta = np.ones(E, np.float32), np.zeros(E, np.float32)
        ref, _ = oracle.tsa_fwd(x, wq, wk, wv, wo, B, S, H, W, scale, causal, tm, True, True, gamma, beta,
                                bq, bk, bv, None, None)
        gref = oracle.tsa_bwd(x, wq, wk, wv, wo, dy, B, S, H, W, scale, causal, tm, bq, bk, bv, None)
        args = tuple(_dev(a) for a in (x, wq, wk, wv, wo))
        kw = dict(scale=scale, causal=causal, time_major=tm, mode=mode)
        use_saved, use_cache = rng.random() < 0.5, rng.random() < 0.5
        saved = ctx.tsa_saved_buffer(*args, B, S, H, W, mode=mode, causal=causal) if use_saved else None
        cache = ctx.tsa_weight_cache(*args, B, S, H, W, mode=mode, causal=causal) if use_cache else None
        out = ctx.tsa_fwd(*args, B, S, H, W, gamma=_dev(gamma), beta=_dev(beta), bq=_dev(bq), bk=_dev(bk),
                          bv=_dev(bv), saved=saved, weight_cache=(cache, False) if use_cache else None, **kw)
        got = ctx.tsa_bwd(*args, _dev(dy), B, S, H, W, bq=_dev(bq), bk=_dev(bk), bv=_dev(bv), saved=saved,
                          reuse_forward=use_saved, weight_cache=(cache, True) if use_cache else None, **kw)
        torch.cuda.synchronize()
        what = (B, S, E, H, W, mode, causal, tm, biases, use_saved, use_cache)
        assert ctx.device_status() == 0, what
        tol = 2e-4 if mode == _lib.MODE_FP32 else 3e-2
        assert rel_l2(out.cpu().numpy(), ref) < tol, what
        for g, r in zip(got, gref):
            assert np.abs(g.cpu().numpy() - r).max() <= tol * max(1.0, np.abs(r).max()), what
        done += 1
