"""The reference's FlashAttention module (src/ml/flash_attention.cu:808-1150): LayerNorm on the input,
projections with biases, attention with scale 1/sqrt(head_dim), score clamp 10 and an optional keep-mask,
output projection, residual with the raw input, inverted dropout - through ltca_tsa_fwd with pre_norm set, and
its backward (an extension, the reference class has none) through ltca_tsa_bwd."""
import math

import numpy as np
import pytest

import oracle


def make(B, S, E, H, D, seed, mask):
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((B * S, E)).astype(np.float32)
    dy = rng.standard_normal((B * S, E)).astype(np.float32)
    lim = math.sqrt(6.0 / (E + H * D))
    wq, wk, wv = (rng.uniform(-lim, lim, (E, H * D)).astype(np.float32) for _ in range(3))
    wo = rng.uniform(-lim, lim, (H * D, E)).astype(np.float32)
    biases = tuple((0.1 * rng.standard_normal(n)).astype(np.float32) for n in (H * D, H * D, H * D, E))
    gamma = (1.0 + 0.1 * rng.standard_normal(E)).astype(np.float32)
    beta = (0.1 * rng.standard_normal(E)).astype(np.float32)
    m = None
    if mask:
        m = (rng.uniform(size=(B, S, S)) < 0.8).astype(np.float32)
        m[:, np.arange(S), np.arange(S)] = 1.0
    return x, dy, wq, wk, wv, wo, biases, gamma, beta, m


def test_oracle_backward_matches_finite_differences():
    B, S, E, H, D = 2, 5, 12, 2, 4
    x, dy, wq, wk, wv, wo, biases, gamma, beta, m = make(B, S, E, H, D, 1, True)
    kw = dict(biases=biases, gamma=gamma, beta=beta, keep_mask=m, dropout_prob=0.25, dropout_seed=7)
    g = oracle.fa_bwd(x, wq, wk, wv, wo, dy, B, S, H, D, **kw)
    f = lambda xx: float((oracle.fa_fwd(xx, wq, wk, wv, wo, B, S, H, D, **kw) * dy).sum())
    x64 = x.astype(np.float64)
    for idx in ((0, 0), (3, 5), (9, 11)):
        xp, xm = x64.copy(), x64.copy()
        xp[idx] += 1e-3
        xm[idx] -= 1e-3
        assert abs((f(xp) - f(xm)) / 2e-3 - g["dx"][idx]) < 2e-3
    keep = oracle.dropout_keep(7, 200000, 0.25)
    assert abs(keep.mean() - 0.75) < 5e-3


FA_CASES = [
    # B, S, E, H, D, mask, dropout, layer_norm, residual, mode, tolerance
    (2, 8, 32, 2, 16, False, 0.0, True, True, "fp32", 2e-4),      # the reference's test fixture shape
    (2, 16, 64, 4, 16, True, 0.1, True, True, "fp32", 2e-4),
    (3, 40, 48, 3, 8, True, 0.3, False, True, "fp32", 2e-4),
    (2, 24, 32, 2, 16, False, 0.0, True, False, "fp32", 2e-4),
    # tensor-pipe mode: every operand of a bf16 tensor-core product is rounded to bf16 (up to 2^-8 relative each);
    # the oracle is fed the bf16-rounded weights and output gradient, and the result is held to two stacked
    # worst-case roundings, 2^-7 of the largest magnitude (the derivation is in tests/test_configs_gpu.py)
    (4, 128, 256, 4, 64, False, 0.1, True, True, "tensor", 2.0 ** -7),
]


@pytest.mark.gpu
@pytest.mark.parametrize("case", FA_CASES)
def test_cuda_flash_attention_module(ctx, case):
    import torch
    from cuda_ltc_b200 import _lib
    B, S, E, H, D, mask, p, ln, res, mode, tol = case
    x, dy, wq, wk, wv, wo, biases, gamma, beta, m = make(B, S, E, H, D, 5, mask)
    kw = dict(biases=biases, gamma=gamma, beta=beta, use_layer_norm=ln, use_residual=res, keep_mask=m,
              dropout_prob=p, dropout_seed=99)
    if mode == "tensor":
        from util import bf16_round
        ref = oracle.fa_fwd(x, *(bf16_round(w) for w in (wq, wk, wv, wo)), B, S, H, D, **kw)
        gref = oracle.fa_bwd(x, *(bf16_round(w) for w in (wq, wk, wv, wo)), bf16_round(dy), B, S, H, D, **kw)
    else:
        ref = oracle.fa_fwd(x, wq, wk, wv, wo, B, S, H, D, **kw)
        gref = oracle.fa_bwd(x, wq, wk, wv, wo, dy, B, S, H, D, **kw)
    dev = lambda a: None if a is None else torch.from_numpy(a).cuda()
    dkw = dict(biases=tuple(dev(b) for b in biases), gamma=dev(gamma), beta=dev(beta), use_layer_norm=ln,
               use_residual=res, keep_mask=dev(m), dropout_prob=p, dropout_seed=99,
               mode=_lib.MODE_FP32 if mode == "fp32" else _lib.MODE_BF16)
    args = (dev(x), dev(wq), dev(wk), dev(wv), dev(wo))
    out = ctx.fa_fwd(*args, B, S, H, D, **dkw)
    got = ctx.fa_bwd(*args, dev(dy), B, S, H, D, **dkw)
    again = ctx.fa_bwd(*args, dev(dy), B, S, H, D, **dkw)
    torch.cuda.synchronize()
    assert ctx.device_status() == 0
    assert np.abs(out.cpu().numpy() - ref).max() < tol * max(1.0, np.abs(ref).max())
    # dropped elements are exactly zero and in the same places
    if p > 0:
        assert ((out.cpu().numpy() == 0) == (ref == 0)).all()
    # the key bias shifts every score of a row by the same amount, so its exact gradient is zero: the three
    # projection-bias gradients (sums of the same kind over the same rows) share one magnitude for the tolerance
    bias_mag = max(float(np.abs(gref[n]).max()) for n in ("dbq", "dbk", "dbv"))
    for name, r in gref.items():
        g = got[name].cpu().numpy()
        assert torch.equal(got[name], again[name]), f"{name}: two runs differ"
        mag = bias_mag if name in ("dbq", "dbk", "dbv") else float(np.abs(r).max())
        assert np.abs(g - r).max() < tol * max(1.0, mag), f"{name}: {np.abs(g - r).max()} vs {mag}"
