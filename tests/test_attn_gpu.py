"""GPU parity tests of the attention core, through the C ABI, against the fp64 oracle.

Tolerances (north_star): fp32 mode max-abs 1e-5; tensor-pipe (bf16 operand) mode max-abs 2e-3
and rel-L2 1e-3, with the oracle consuming the bf16-rounded inputs.  When the OUTPUT is stored
as bf16 its own rounding (half an ulp = 2^-9 relative) is allowed on top, and written as such.
"""
import math

import numpy as np
import pytest
import torch

import oracle
from cuda_ltc_b200 import _lib
from util import bf16_round, keep_mask, max_abs, randn, rel_l2

pytestmark = pytest.mark.gpu

FP32_TOL = 1e-5
TC_MAX_ABS, TC_REL_L2 = 2e-3, 1e-3


def dev(a, dtype=torch.float32):
    return torch.from_numpy(np.ascontiguousarray(a)).to("cuda", dtype)


def make_case(B, H, Sq, Sk, D, seed, scale_in=1.0):
    q = randn((B, H, Sq, D), seed, scale_in)
    k = randn((B, H, Sk, D), seed + 1, scale_in)
    v = randn((B, H, Sk, D), seed + 2, scale_in)
    do = randn((B, H, Sq, D), seed + 3, scale_in)
    return q, k, v, do


FP32_CASES = [
    # B, H, Sq, Sk, D, causal, mask, kvlen, clamp
    (2, 4, 64, 64, 32, False, False, False, 0.0),      # config 1 of the benchmark
    (2, 2, 8, 8, 16, False, False, False, 10.0),       # the reference test fixture
    (2, 4, 16, 16, 16, True, True, False, 10.0),
    (1, 2, 1, 1, 16, False, False, False, 0.0),
    (1, 2, 7, 7, 20, True, False, False, 0.0),
    (2, 1, 17, 17, 64, True, False, True, 0.0),
    (1, 2, 129, 129, 128, True, False, False, 0.0),
    (2, 2, 33, 70, 24, False, True, True, 0.7),
    (1, 1, 70, 33, 8, True, False, False, 0.0),        # more queries than keys: early rows see nothing
    (2, 8, 256, 256, 64, True, False, False, 0.0),     # per-head shape of config 2
    (2, 2, 32, 32, 512, False, False, False, 0.0),     # wide heads: the reference module's head width = model width
    (1, 3, 50, 77, 200, True, True, True, 2.0),        # wide, every mask kind, ragged width
    (2, 1, 40, 24, 256, True, False, False, 0.0),      # wide, more queries than keys
]


@pytest.mark.parametrize("case", FP32_CASES)
def test_fp32_forward_backward(ctx, case):
    B, H, Sq, Sk, D, causal, use_mask, use_len, clamp = case
    q, k, v, do = make_case(B, H, Sq, Sk, D, 100)
    m = keep_mask(B, Sq, Sk, 5) if use_mask else None
    L = np.random.default_rng(6).integers(0, Sk + 1, size=B).astype(np.int32) if use_len else None
    sc = 1.0 / math.sqrt(D)
    o_ref, lse_ref = oracle.attn_fwd(q, k, v, sc, causal, m, L, clamp)
    dm = dev(m) if m is not None else None
    dL = torch.from_numpy(L).cuda() if L is not None else None
    tq, tk, tv, tdo = dev(q), dev(k), dev(v), dev(do)
    o, lse = ctx.attn_fwd(tq, tk, tv, scale=sc, causal=causal, keep_mask=dm, kv_len=dL,
                          score_clamp=clamp, mode=_lib.MODE_FP32)
    assert max_abs(o.cpu().numpy(), o_ref) < FP32_TOL
    lse_h = lse.cpu().numpy().astype(np.float64)
    fin = np.isfinite(lse_ref)
    assert (np.isfinite(lse_h) == fin).all()
    assert max_abs(lse_h[fin], lse_ref[fin]) < 1e-5
    dq_ref, dk_ref, dv_ref = oracle.attn_bwd(q, k, v, do, sc, causal, m, L, clamp)
    dq, dk, dv = ctx.attn_bwd(tq, tk, tv, o, lse, tdo, scale=sc, causal=causal, keep_mask=dm,
                              kv_len=dL, score_clamp=clamp, mode=_lib.MODE_FP32)
    for got, ref in ((dq, dq_ref), (dk, dk_ref), (dv, dv_ref)):
        assert max_abs(got.cpu().numpy(), ref) < FP32_TOL * max(1.0, float(np.abs(ref).max()))


def test_fp32_strided_projection_layout(ctx):
    """q, k, v addressed in place inside a [B*S, 3*H*D] projection buffer (no reshape copies)."""
    B, H, S, D = 2, 4, 40, 32
    x = randn((B, S, 3, H, D), 7)
    tx = dev(x)
    views = [tx[:, :, i].permute(0, 2, 1, 3) for i in range(3)]
    o, _ = ctx.attn_fwd(*views, causal=True, mode=_lib.MODE_FP32)
    o_ref, _ = oracle.attn_fwd(*(x[:, :, i].transpose(0, 2, 1, 3) for i in range(3)), 1 / math.sqrt(D), True)
    assert max_abs(o.cpu().numpy(), o_ref) < FP32_TOL


def test_fp32_backward_is_repeatable(ctx):
    """The reference pins backward repeatability at 1e-6 (time_self_attention_test.cu:799-838);
    the fp32 backward has no atomics, so two runs agree bit for bit."""
    q, k, v, do = (dev(a) for a in make_case(2, 2, 100, 100, 32, 300))
    o, lse = ctx.attn_fwd(q, k, v, causal=True, mode=_lib.MODE_FP32)
    a = ctx.attn_bwd(q, k, v, o, lse, do, causal=True, mode=_lib.MODE_FP32)
    b = ctx.attn_bwd(q, k, v, o, lse, do, causal=True, mode=_lib.MODE_FP32)
    for x, y in zip(a, b):
        assert torch.equal(x, y)


TC_CASES = [
    # B, H, Sq, Sk, D, causal, kvlen, mask, clamp
    (1, 1, 128, 128, 64, False, False, False, 0.0),
    (1, 2, 256, 256, 64, True, False, False, 0.0),
    (2, 2, 384, 384, 64, True, False, False, 0.0),
    (2, 3, 257, 257, 64, True, False, False, 0.0),
    (1, 2, 1000, 1000, 64, False, True, False, 0.0),
    (2, 2, 130, 515, 64, True, True, False, 0.0),
    (1, 2, 200, 200, 64, True, False, True, 5.0),
    (32, 8, 256, 256, 64, True, False, False, 0.0),     # config 2 core
    (1, 2, 512, 512, 128, True, False, False, 0.0),
    (1, 1, 300, 300, 128, False, True, False, 0.0),
    # few (batch, head) pairs and long query ranges: the two-tile kernel over several 256-row blocks (the
    # four-tile kernel's 512-row work items would leave most SMs idle)
    (1, 2, 1100, 1100, 64, True, False, False, 0.0),
    (2, 2, 2048, 2048, 64, True, False, False, 0.0),
    (1, 3, 1536, 1000, 64, True, False, False, 0.0),    # more queries than keys: the early tiles see nothing
    (1, 2, 1000, 1500, 64, True, True, False, 0.0),     # key lengths
    (1, 2, 640, 640, 64, True, False, True, 5.0),       # dense mask and clamp
    # enough pairs that the four-tile kernel's items fill the SMs about as well, and still no more items than SMs:
    # causal launches take its folded tile mapping (two early and two late query tiles per item)
    (5, 8, 1100, 1100, 64, True, False, False, 0.0),    # nine tiles in three blocks: three padded tile slots
    (4, 8, 2048, 2048, 64, True, False, False, 0.0),
    (5, 8, 1536, 1000, 64, True, False, False, 0.0),
    (5, 8, 1000, 1500, 64, True, True, False, 0.0),
    (8, 8, 640, 640, 64, True, False, True, 5.0),
    (10, 16, 512, 700, 64, False, True, False, 0.0),    # more items than SMs: the plain mapping, items from a queue
]


@pytest.mark.parametrize("storage", ["bf16", "f32"])
@pytest.mark.parametrize("case", TC_CASES)
def test_tensor_pipe_forward(ctx, case, storage):
    B, H, Sq, Sk, D, causal, use_len, use_mask, clamp = case
    q, k, v, _ = make_case(B, H, Sq, Sk, D, 200, 0.5 if storage == "bf16" else 1.0)
    qr, kr, vr = bf16_round(q), bf16_round(k), bf16_round(v)
    L = np.random.default_rng(8).integers(1, Sk + 1, size=B).astype(np.int32) if use_len else None
    m = keep_mask(B, Sq, Sk, 9, 0.8, dead_rows=((0, 3),)) if use_mask else None
    sc = 1.0 / math.sqrt(D)
    o_ref, lse_ref = oracle.attn_fwd(qr, kr, vr, sc, causal, m, L, clamp)
    dt = torch.bfloat16 if storage == "bf16" else torch.float32
    tq, tk, tv = dev(q, dt), dev(k, dt), dev(v, dt)
    dL = torch.from_numpy(L).cuda() if L is not None else None
    dm = dev(m) if m is not None else None
    assert ctx.uses_tensor_pipe(tq, tk, tv, causal=causal, mode=_lib.MODE_BF16)
    o, lse = ctx.attn_fwd(tq, tk, tv, scale=sc, causal=causal, kv_len=dL, keep_mask=dm,
                          score_clamp=clamp, mode=_lib.MODE_BF16)
    torch.cuda.synchronize()
    assert ctx.device_status() == 0
    got = o.float().cpu().numpy()
    err = np.abs(got.astype(np.float64) - o_ref)
    if storage == "bf16":
        allowed = TC_MAX_ABS + np.abs(o_ref) * 2.0 ** -8     # + half-ulp of the bf16 output
        assert (err <= allowed).all(), f"max excess {(err - allowed).max()}"
        assert rel_l2(got, o_ref) < TC_REL_L2 + 2.0 ** -9
    else:
        assert err.max() < TC_MAX_ABS
        assert rel_l2(got, o_ref) < TC_REL_L2
    lse_h = lse.cpu().numpy().astype(np.float64)
    fin = np.isfinite(lse_ref)
    assert (np.isfinite(lse_h) == fin).all()
    assert max_abs(lse_h[fin], lse_ref[fin]) < 2e-3


def test_tensor_pipe_full_size_properties(ctx):
    """Config 3 (B=8 H=16 S=4096 D=64 causal bf16) at full size: size-independent properties
    (V = const gives O = const; row 0 returns v_0; lse of row 0 is its single score) plus an
    oracle check of a subset of (batch, head) pairs."""
    B, H, S, D = 8, 16, 4096, 64
    g = torch.Generator(device="cuda").manual_seed(3)
    q = (torch.randn((B, H, S, D), generator=g, device="cuda") * 0.5).bfloat16()
    k = (torch.randn((B, H, S, D), generator=g, device="cuda") * 0.5).bfloat16()
    v = (torch.randn((B, H, S, D), generator=g, device="cuda") * 0.5).bfloat16()
    o, lse = ctx.attn_fwd(q, k, v, causal=True, mode=_lib.MODE_BF16)
    torch.cuda.synchronize()
    assert ctx.device_status() == 0
    assert torch.equal(o[:, :, 0], v[:, :, 0])
    s00 = (q[:, :, 0].float() * k[:, :, 0].float()).sum(-1) / 8.0
    assert (lse[:, :, 0] - s00).abs().max().item() < 1e-3
    ones = torch.ones_like(v)
    o1, _ = ctx.attn_fwd(q, k, ones, causal=True, mode=_lib.MODE_BF16)
    assert (o1.float() - 1.0).abs().max().item() <= 2.0 ** -7
    for (b, h) in ((0, 0), (3, 7), (7, 15)):
        qs, ks, vs = (t[b:b + 1, h:h + 1].float().cpu().numpy() for t in (q, k, v))
        o_ref, lse_ref = oracle.attn_fwd(qs, ks, vs, 0.125, True)
        got = o[b, h].float().cpu().numpy()[None, None]
        err = np.abs(got - o_ref)
        assert (err <= TC_MAX_ABS + np.abs(o_ref) * 2.0 ** -8).all()
        assert max_abs(lse[b, h].cpu().numpy()[None, None], lse_ref) < 2e-3


DECODE_CASES = [
    # B, H, Smax, D, dtype, mask
    (256, 8, 1024, 64, torch.float32, False),     # config 4
    (3, 2, 77, 16, torch.float32, True),
    (2, 4, 300, 32, torch.float32, False),
    (2, 2, 2048, 128, torch.float32, False),      # few (batch, head) pairs: split over keys
    (4, 8, 512, 64, torch.bfloat16, False),
]


@pytest.mark.parametrize("case", DECODE_CASES)
def test_decode(ctx, case):
    B, H, Smax, D, dt, use_mask = case
    q, k, v, _ = make_case(B, H, 1, Smax, D, 400)
    if dt == torch.bfloat16:
        q, k, v = bf16_round(q), bf16_round(k), bf16_round(v)
    L = np.random.default_rng(10).integers(1, Smax + 1, size=B).astype(np.int32)
    L[0] = Smax
    if B > 2:
        L[1] = 1
    m = keep_mask(B, 1, Smax, 11, 0.6, dead_rows=()) if use_mask else None
    sc = 1.0 / math.sqrt(D)
    o_ref, lse_ref = oracle.attn_fwd(q, k, v, sc, False, m, L)
    o, lse = ctx.attn_decode(dev(q, dt), dev(k, dt), dev(v, dt), kv_len=torch.from_numpy(L).cuda(),
                             scale=sc, keep_mask=dev(m) if m is not None else None)
    tol = FP32_TOL if dt == torch.float32 else 2.0 ** -8
    assert max_abs(o.float().cpu().numpy(), o_ref) < tol * max(1.0, float(np.abs(o_ref).max()))
    lse_h = lse.cpu().numpy().astype(np.float64)
    fin = np.isfinite(lse_ref)
    assert (np.isfinite(lse_h) == fin).all()
    assert max_abs(lse_h[fin], lse_ref[fin]) < 1e-5 * max(1.0, float(np.abs(lse_ref[fin]).max()))


def test_decode_zero_length(ctx):
    B, H, Smax, D = 2, 2, 64, 64
    q, k, v, _ = (dev(a) for a in make_case(B, H, 1, Smax, D, 500))
    L = torch.tensor([0, 5], dtype=torch.int32, device="cuda")
    o, lse = ctx.attn_decode(q, k, v, kv_len=L)
    assert (o[0] == 0).all() and torch.isneginf(lse[0]).all() and torch.isfinite(lse[1]).all()


def test_argument_errors(ctx):
    from cuda_ltc_b200 import LtcaError
    q = torch.zeros((1, 1, 4, 20), device="cuda")
    with pytest.raises(LtcaError) as e:
        ctx.attn_fwd(q, q, q, mode=_lib.MODE_BF16)       # head_dim 20: no tensor path takes rows that are not 16-byte multiples
    assert e.value.code == -2
    with pytest.raises(LtcaError) as e:
        ctx.attn_fwd(q, q, q, scale=-1.0)
    assert e.value.code == -1
    big = torch.zeros((1, 1, 4, 1024), device="cuda")        # wider than the widest head the exact kernels take (512)
    with pytest.raises(LtcaError):
        ctx.attn_fwd(big, big, big, mode=_lib.MODE_FP32)


TC_BWD_CASES = [
    # B, H, Sq, Sk, causal, kvlen, mask, clamp      (head_dim 64)
    (1, 1, 128, 128, False, False, False, 0.0),
    (1, 2, 256, 256, True, False, False, 0.0),
    (2, 2, 384, 384, True, False, False, 0.0),
    (2, 3, 257, 257, True, False, False, 0.0),
    (1, 2, 1000, 1000, False, True, False, 0.0),
    (2, 2, 130, 515, True, True, False, 0.0),
    (1, 2, 200, 200, True, False, True, 5.0),
    (1, 2, 515, 130, True, False, False, 0.0),      # early queries see no key at all
    (32, 8, 256, 256, True, False, False, 0.0),     # config 2 core
    # longer query ranges with every kind of mask
    (1, 2, 640, 640, True, False, True, 5.0),       # dense mask and clamp
    (2, 2, 600, 515, True, True, False, 0.0),       # key lengths, causal, more queries than keys
    (2, 3, 769, 769, True, False, False, 0.0),      # ragged edges
]


@pytest.mark.parametrize("storage", ["bf16", "f32"])
@pytest.mark.parametrize("case", TC_BWD_CASES)
def test_tensor_pipe_backward(ctx, case, storage):
    B, H, Sq, Sk, causal, use_len, use_mask, clamp = case
    D = 64
    q, k, v, do = make_case(B, H, Sq, Sk, D, 600, 0.5 if storage == "bf16" else 1.0)
    qr, kr, vr, dor = bf16_round(q), bf16_round(k), bf16_round(v), bf16_round(do)
    L = np.random.default_rng(8).integers(1, Sk + 1, size=B).astype(np.int32) if use_len else None
    m = keep_mask(B, Sq, Sk, 9, 0.8, dead_rows=((0, 3),)) if use_mask else None
    sc = 1.0 / math.sqrt(D)
    ref = oracle.attn_bwd(qr, kr, vr, dor, sc, causal, m, L, clamp)
    dt = torch.bfloat16 if storage == "bf16" else torch.float32
    tq, tk, tv, tdo = dev(q, dt), dev(k, dt), dev(v, dt), dev(do, dt)
    dL = torch.from_numpy(L).cuda() if L is not None else None
    dm = dev(m) if m is not None else None
    kw = dict(scale=sc, causal=causal, kv_len=dL, keep_mask=dm, score_clamp=clamp, mode=_lib.MODE_BF16)
    assert ctx.uses_tensor_pipe(tq, tk, tv, causal=causal, mode=_lib.MODE_BF16, backward=True)
    o, lse = ctx.attn_fwd(tq, tk, tv, **kw)
    got = ctx.attn_bwd(tq, tk, tv, o, lse, tdo, **kw)
    again = ctx.attn_bwd(tq, tk, tv, o, lse, tdo, **kw)
    det = ctx.attn_bwd(tq, tk, tv, o, lse, tdo, deterministic=True, **kw)
    det_again = ctx.attn_bwd(tq, tk, tv, o, lse, tdo, deterministic=True, **kw)
    torch.cuda.synchronize()
    assert ctx.device_status() == 0
    for name, g, g2 in zip(("dq", "dk", "dv"), det, det_again):
        assert torch.equal(g, g2), f"{name}: two deterministic runs differ"     # no atomics on that path
    for name, g, g2 in zip(("dq", "dk", "dv"), got, again):
        if name == "dq" and storage == "bf16":
            # fused kernel: the key blocks' shares of dQ are added in fp32 in no fixed order, then rounded once to
            # bf16: two runs agree to that rounding (one ulp = 2^-7 relative on the rare element that flips)
            a32, b32 = g.float(), g2.float()
            assert ((a32 - b32).abs() <= 2.0 ** -7 * b32.abs() + 1e-6).all(), "dq: runs differ by more than one ulp"
        else:
            assert torch.equal(g, g2), f"{name}: two runs differ"
    for name, g, r in [(n, g, r) for n, g, r in zip(("dq", "dk", "dv"), got, ref)] + \
                      [(n + " (deterministic)", g, r) for n, g, r in zip(("dq", "dk", "dv"), det, ref)]:
        gh = g.float().cpu().numpy().astype(np.float64)
        mag = max(1.0, float(np.abs(r).max()))
        err = np.abs(gh - r)
        if storage == "bf16":
            allowed = TC_MAX_ABS * mag + np.abs(r) * 2.0 ** -8
            assert (err <= allowed).all(), f"{name}: max excess {(err - allowed).max()}"
            assert rel_l2(gh, r) < 2 * (TC_REL_L2 + 2.0 ** -9), name
        else:
            assert err.max() < TC_MAX_ABS * mag, f"{name}: max-abs {err.max()}"
            assert rel_l2(gh, r) < 2 * TC_REL_L2, f"{name}: rel-L2 {rel_l2(gh, r)}"


def test_tensor_pipe_backward_full_size(ctx):
    """Config 3 (B=8 H=16 S=4096 D=64 causal bf16) at full size, backward: two (batch, head) pairs against the
    oracle, bit-identical repeat, and two size-independent properties - the gradient of the last key's value row
    is (its attention weight from the last query) x dO of that query alone, and dO = 0 for one head gives zero
    gradients for that head only."""
    B, H, S, D = 8, 16, 4096, 64
    g = torch.Generator(device="cuda").manual_seed(5)
    mk = lambda: (torch.randn((B, H, S, D), generator=g, device="cuda") * 0.5).bfloat16()
    q, k, v, do = mk(), mk(), mk(), mk()
    do[2, 3] = 0
    o, lse = ctx.attn_fwd(q, k, v, causal=True, mode=_lib.MODE_BF16)
    dq, dk, dv = ctx.attn_bwd(q, k, v, o, lse, do, causal=True, mode=_lib.MODE_AUTO)
    dq2, dk2, dv2 = ctx.attn_bwd(q, k, v, o, lse, do, causal=True, mode=_lib.MODE_AUTO)
    dq3, dk3, dv3 = ctx.attn_bwd(q, k, v, o, lse, do, causal=True, mode=_lib.MODE_AUTO, deterministic=True)
    dq4, dk4, dv4 = ctx.attn_bwd(q, k, v, o, lse, do, causal=True, mode=_lib.MODE_AUTO, deterministic=True)
    torch.cuda.synchronize()
    assert ctx.device_status() == 0
    # fused kernel: dK and dV bit-identical, dQ to the rounding of its fp32 sum; two-kernel path: every bit
    assert torch.equal(dk, dk2) and torch.equal(dv, dv2)
    assert ((dq.float() - dq2.float()).abs() <= 2.0 ** -7 * dq2.float().abs() + 1e-6).all()
    assert torch.equal(dq3, dq4) and torch.equal(dk3, dk4) and torch.equal(dv3, dv4)
    assert torch.equal(dk, dk3) and torch.equal(dv, dv3)        # the same arithmetic for dK and dV on both paths
    assert ((dq.float() - dq3.float()).abs() <= 2.0 ** -6 * dq3.float().abs() + 1e-5).all()
    for t in (dq, dk, dv):
        assert (t[2, 3] == 0).all() and (t[2, 4] != 0).any()
    # the last key is seen by the last query only: dV[S-1] = P[S-1, S-1] * dO[S-1]
    s_last = (q[:, :, -1].float() * k[:, :, -1].float()).sum(-1) / 8.0
    p_last = torch.exp(s_last - lse[:, :, -1])
    want = p_last[..., None] * do[:, :, -1].float()
    assert (dv[:, :, -1].float() - want).abs().max().item() < 2e-3
    for (b, h) in ((0, 0), (7, 15)):
        qs, ks, vs, gs = (t[b:b + 1, h:h + 1].float().cpu().numpy() for t in (q, k, v, do))
        ref = oracle.attn_bwd(qs, ks, vs, gs, 0.125, True)
        for name, got, r in zip(("dq", "dk", "dv"), (dq, dk, dv), ref):
            gh = got[b, h].float().cpu().numpy()[None, None].astype(np.float64)
            mag = max(1.0, float(np.abs(r).max()))
            assert (np.abs(gh - r) <= TC_MAX_ABS * mag + np.abs(r) * 2.0 ** -8).all(), name
            assert rel_l2(gh, r) < 2 * (TC_REL_L2 + 2.0 ** -9), name


WIDE_CORE_CASES = [
    # B, H, Sq, Sk, D, causal, kvlen, mask, clamp
    (2, 4, 64, 64, 32, False, False, False, 0.0),      # config 1 of the benchmark on the tensor pipe
    (2, 2, 8, 8, 16, False, False, False, 10.0),       # the reference test fixture
    (3, 2, 100, 130, 32, True, True, True, 3.0),
    (2, 2, 200, 200, 256, True, False, False, 0.0),
    (1, 2, 70, 33, 8, True, False, False, 0.0),        # more queries than keys: early rows see nothing
    (2, 2, 300, 300, 128, True, False, False, 0.0),    # width 128 backward (no streaming kernel)
]


@pytest.mark.parametrize("storage", ["bf16", "f32"])
@pytest.mark.parametrize("case", WIDE_CORE_CASES)
def test_tensor_pipe_other_head_widths(ctx, case, storage):
    """LTCA_MODE_BF16 with a head width the streaming kernels do not cover (any multiple of 8): written-out
    scores and batched tcgen05 GEMMs.  Same arithmetic class as the streaming bf16 mode (bf16 operands, fp32
    accumulation, P and dS rounded once to bf16), hence the same tolerances."""
    B, H, Sq, Sk, D, causal, use_len, use_mask, clamp = case
    q, k, v, do = make_case(B, H, Sq, Sk, D, 700, 0.5 if storage == "bf16" else 1.0)
    qr, kr, vr, dor = bf16_round(q), bf16_round(k), bf16_round(v), bf16_round(do)
    L = np.random.default_rng(8).integers(1, Sk + 1, size=B).astype(np.int32) if use_len else None
    m = keep_mask(B, Sq, Sk, 9, 0.8, dead_rows=((0, 3),)) if use_mask else None
    sc = 1.0 / math.sqrt(D)
    o_ref, lse_ref = oracle.attn_fwd(qr, kr, vr, sc, causal, m, L, clamp)
    ref = oracle.attn_bwd(qr, kr, vr, dor, sc, causal, m, L, clamp)
    dt = torch.bfloat16 if storage == "bf16" else torch.float32
    tq, tk, tv, tdo = dev(q, dt), dev(k, dt), dev(v, dt), dev(do, dt)
    dL = torch.from_numpy(L).cuda() if L is not None else None
    dm = dev(m) if m is not None else None
    kw = dict(scale=sc, causal=causal, kv_len=dL, keep_mask=dm, score_clamp=clamp, mode=_lib.MODE_BF16)
    if D != 128:
        assert ctx.uses_tensor_pipe(tq, tk, tv, causal=causal, mode=_lib.MODE_BF16)
    assert ctx.uses_tensor_pipe(tq, tk, tv, causal=causal, mode=_lib.MODE_BF16, backward=True)
    o, lse = ctx.attn_fwd(tq, tk, tv, **kw)
    got = ctx.attn_bwd(tq, tk, tv, o, lse, tdo, **kw)
    again = ctx.attn_bwd(tq, tk, tv, o, lse, tdo, **kw)
    torch.cuda.synchronize()
    assert ctx.device_status() == 0
    half_ulp = 2.0 ** -8 if storage == "bf16" else 0.0
    oh = o.float().cpu().numpy().astype(np.float64)
    assert (np.abs(oh - o_ref) <= TC_MAX_ABS + np.abs(o_ref) * half_ulp).all(), np.abs(oh - o_ref).max()
    assert rel_l2(oh, o_ref) < TC_REL_L2 + half_ulp / 2
    lse_h = lse.cpu().numpy().astype(np.float64)
    fin = np.isfinite(lse_ref)
    assert (np.isfinite(lse_h) == fin).all()
    assert max_abs(lse_h[fin], lse_ref[fin]) < 2e-3
    for name, g, g2, r in zip(("dq", "dk", "dv"), got, again, ref):
        assert torch.equal(g, g2), f"{name}: two runs differ"
        gh = g.float().cpu().numpy().astype(np.float64)
        mag = max(1.0, float(np.abs(r).max()))
        assert (np.abs(gh - r) <= TC_MAX_ABS * mag + np.abs(r) * half_ulp).all(), name
        assert rel_l2(gh, r) < 2 * (TC_REL_L2 + half_ulp / 2), f"{name}: rel-L2 {rel_l2(gh, r)}"


# Two bf16 terms carry 16 significant bits: a value x is represented to within 2^-17 |x|, so an output row that is
# a mix of a few large values of v (a causal row that sees one or two keys) is off by that fraction of THEIR size,
# whatever its own size; on top of it the sums contribute an absolute part.  Measured at these shapes: 1e-5 .. 6e-5 max-abs, 6e-6 .. 9e-6 relative L2
# (the exact fp32 mode: 1e-6, the bf16 mode: 6e-3).
SPLIT_ABS = 2e-5
SPLIT_REL = 2.0 ** -16
SPLIT_REL_L2 = 2e-5


@pytest.mark.parametrize("case", WIDE_CORE_CASES + [(2, 2, 200, 200, 64, True, False, False, 0.0),
                                                    (1, 2, 640, 515, 64, True, True, False, 0.0)])
def test_split_precision_mode(ctx, case):
    """LTCA_MODE_SPLIT: fp32 storage on the tensor pipe with every operand (Q, K, V, dO, P, dS) as two bf16 terms
    and three-term products.  Sixteen significant bits per operand - TF32 keeps eleven - give agreement with the
    fp64 oracle ON THE EXACT INPUTS at the 1e-5 level, two hundred times tighter than the bf16 mode, at every head
    width that is a multiple of 8."""
    B, H, Sq, Sk, D, causal, use_len, use_mask, clamp = case
    q, k, v, do = make_case(B, H, Sq, Sk, D, 900, 1.0)
    L = np.random.default_rng(8).integers(1, Sk + 1, size=B).astype(np.int32) if use_len else None
    m = keep_mask(B, Sq, Sk, 9, 0.8, dead_rows=((0, 3),)) if use_mask else None
    sc = 1.0 / math.sqrt(D)
    o_ref, lse_ref = oracle.attn_fwd(q, k, v, sc, causal, m, L, clamp)
    ref = oracle.attn_bwd(q, k, v, do, sc, causal, m, L, clamp)
    tq, tk, tv, tdo = dev(q, torch.float32), dev(k, torch.float32), dev(v, torch.float32), dev(do, torch.float32)
    dL = torch.from_numpy(L).cuda() if L is not None else None
    dm = dev(m) if m is not None else None
    kw = dict(scale=sc, causal=causal, kv_len=dL, keep_mask=dm, score_clamp=clamp, mode=_lib.MODE_SPLIT)
    assert ctx.uses_tensor_pipe(tq, tk, tv, causal=causal, mode=_lib.MODE_SPLIT)
    assert ctx.uses_tensor_pipe(tq, tk, tv, causal=causal, mode=_lib.MODE_SPLIT, backward=True)
    o, lse = ctx.attn_fwd(tq, tk, tv, **kw)
    got = ctx.attn_bwd(tq, tk, tv, o, lse, tdo, **kw)
    again = ctx.attn_bwd(tq, tk, tv, o, lse, tdo, **kw)
    torch.cuda.synchronize()
    assert ctx.device_status() == 0
    oh = o.cpu().numpy().astype(np.float64)
    assert np.abs(oh - o_ref).max() <= SPLIT_ABS + SPLIT_REL * np.abs(v).max(), np.abs(oh - o_ref).max()
    assert rel_l2(oh, o_ref) < SPLIT_REL_L2
    lse_h = lse.cpu().numpy().astype(np.float64)
    fin = np.isfinite(lse_ref)
    assert (np.isfinite(lse_h) == fin).all()
    assert (np.abs(lse_h[fin] - lse_ref[fin]) <= SPLIT_ABS + SPLIT_REL * np.abs(lse_ref[fin])).all()
    for name, g, g2, r in zip(("dq", "dk", "dv"), got, again, ref):
        assert torch.equal(g, g2), f"{name}: two runs differ"
        gh = g.cpu().numpy().astype(np.float64)
        mag = max(1.0, float(np.abs(r).max()))
        assert np.abs(gh - r).max() <= (SPLIT_ABS + SPLIT_REL) * mag, (name, np.abs(gh - r).max())
        assert rel_l2(gh, r) < SPLIT_REL_L2, f"{name}: rel-L2 {rel_l2(gh, r)}"


def test_host_step_pipeline_matches_direct_calls(ctx):
    """Operands in pinned host memory, results back to pinned host memory, three overlapping steps:
    the same bits as the direct device-buffer calls."""
    from cuda_ltc_b200 import HostStepPipeline
    B, H, S, D = 2, 4, 640, 64
    g = torch.Generator(device="cuda").manual_seed(11)
    q, k, v, do = ((torch.randn((B, H, S, D), generator=g, device="cuda") * 0.5).bfloat16() for _ in range(4))
    o, lse = ctx.attn_fwd(q, k, v, causal=True, mode=_lib.MODE_BF16)
    dq, dk, dv = ctx.attn_bwd(q, k, v, o, lse, do, causal=True, mode=_lib.MODE_AUTO, deterministic=True)
    host_in = tuple(t.cpu().pin_memory() for t in (q, k, v, do))
    host_out = tuple(torch.zeros_like(t).pin_memory() for t in host_in)
    stream = torch.cuda.Stream()
    ctx2 = type(ctx)(0, stream)
    pipe = HostStepPipeline(ctx2, stream, q, k, causal=True, deterministic=True)      # bit-identical gradients
    pipe.run(host_in, host_out, 3)
    torch.cuda.synchronize()
    assert ctx2.device_status() == 0
    for got, ref in zip(host_out, (o, dq, dk, dv)):
        assert torch.equal(got, ref.cpu())


def test_sm_limit_changes_the_launch_width_not_the_results(ctx):
    """Capping the SMs the persistent kernels spread over (room for a communication library's kernels)
    must leave forward and backward results bit-identical; 0 restores the default."""
    import torch
    g = torch.Generator(device="cuda").manual_seed(4)
    # (4 x 40 pairs of 512 queries: 160 work items of the persistent forward kernel, more than there are SMs)
    q, k, v, do = ((torch.randn((4, 40, 512, 64), generator=g, device="cuda") * 0.5).bfloat16() for _ in range(4))
    o, lse = ctx.attn_fwd(q, k, v, causal=True)
    grads = ctx.attn_bwd(q, k, v, o, lse, do, causal=True, deterministic=True)
    fused = ctx.attn_bwd(q, k, v, o, lse, do, causal=True)
    try:
        ctx.set_sm_limit(ctx.sm_count() - 40)
        o2, lse2 = ctx.attn_fwd(q, k, v, causal=True)
        grads2 = ctx.attn_bwd(q, k, v, o2, lse2, do, causal=True, deterministic=True)
        fused2 = ctx.attn_bwd(q, k, v, o2, lse2, do, causal=True)
    finally:
        ctx.set_sm_limit(0)
    torch.cuda.synchronize()
    assert ctx.device_status() == 0
    assert torch.equal(o, o2) and torch.equal(lse, lse2)
    for a, b in zip(grads, grads2):
        assert torch.equal(a, b)
    # the fused backward: dK and dV bit-identical, dQ up to the rounding of its unordered fp32 sum
    assert torch.equal(fused[1], fused2[1]) and torch.equal(fused[2], fused2[2])
    assert ((fused[0].float() - fused2[0].float()).abs() <= 2.0 ** -7 * fused2[0].float().abs() + 1e-6).all()


@pytest.mark.gpu
@pytest.mark.parametrize("deterministic", [False, True])
def test_backward_with_runs_of_empty_work_items(ctx, deterministic):
    """More work items than SMs, most of them without work (short key lengths in four of five batch entries, and
    more queries than keys under a causal mask): the persistent backward kernels skip long runs of empty items
    behind an item with work, whose last accumulation must not wait for the next item with work."""
    B, H, Sq, Sk, D = 5, 11, 1062, 865, 64
    q, k, v, do = make_case(B, H, Sq, Sk, D, 610, 0.5)
    qr, kr, vr, dor = bf16_round(q), bf16_round(k), bf16_round(v), bf16_round(do)
    L = np.array([865, 40, 130, 20, 7], dtype=np.int32)
    sc = 1.0 / math.sqrt(D)
    o_ref, lse_ref = oracle.attn_fwd(qr, kr, vr, sc, True, None, L, 0.0)
    ref = oracle.attn_bwd(qr, kr, vr, dor, sc, True, None, L, 0.0)
    tq, tk, tv, tdo = (dev(x, torch.bfloat16) for x in (q, k, v, do))
    dL = torch.from_numpy(L).cuda()
    o, lse = ctx.attn_fwd(tq, tk, tv, scale=sc, causal=True, kv_len=dL, mode=_lib.MODE_BF16)
    grads = ctx.attn_bwd(tq, tk, tv, o, lse, tdo, scale=sc, causal=True, kv_len=dL, mode=_lib.MODE_BF16,
                         deterministic=deterministic)
    torch.cuda.synchronize()
    assert ctx.device_status() == 0
    # (bf16 storage: the stored result carries one more rounding, as in test_tensor_pipe_backward)
    assert (np.abs(o.float().cpu().numpy() - o_ref) <= TC_MAX_ABS + np.abs(o_ref) * 2.0 ** -8).all()
    for got, want in zip(grads, ref):
        gh = got.float().cpu().numpy().astype(np.float64)
        allowed = TC_MAX_ABS * max(1.0, float(np.abs(want).max())) + np.abs(want) * 2.0 ** -8
        assert (np.abs(gh - want) <= allowed).all()
        assert rel_l2(gh, want) < 2 * (TC_REL_L2 + 2.0 ** -9)
