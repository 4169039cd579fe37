"""CPU tests of the oracle: the C restatement against the independent numpy restatement,
against analytic properties, and against the golden vectors produced by the reference's own
kernel (tests/golden/)."""
import glob
import os

import numpy as np
import pytest

import oracle
from util import keep_mask, randn

CASES = [
    # B, H, Sq, Sk, D, causal, mask, kvlen, clamp
    (2, 3, 17, 17, 8, False, False, False, 0.0),
    (2, 2, 16, 16, 16, True, False, False, 10.0),
    (2, 2, 9, 21, 4, True, True, True, 0.5),
    (1, 2, 5, 5, 4, False, True, False, 0.0),
    (2, 4, 64, 64, 32, False, False, False, 0.0),
    (1, 1, 1, 33, 16, False, False, True, 0.0),
]


@pytest.mark.parametrize("case", CASES)
def test_c_matches_numpy(case):
    B, H, Sq, Sk, D, causal, use_mask, use_len, clamp = case
    q, k, v, do = randn((B, H, Sq, D), 1), randn((B, H, Sk, D), 2), randn((B, H, Sk, D), 3), randn((B, H, Sq, D), 4)
    m = keep_mask(B, Sq, Sk, 5) if use_mask else None
    L = np.random.default_rng(6).integers(1, Sk + 1, size=B).astype(np.int32) if use_len else None
    sc = 1.0 / np.sqrt(D)
    o, lse = oracle.attn_fwd(q, k, v, sc, causal, m, L, clamp)
    o2, lse2 = oracle.attn_fwd_numpy(q, k, v, sc, causal, m, L, clamp)
    assert np.abs(o - o2).max() < 1e-12
    fin = np.isfinite(lse2)
    assert (np.isfinite(lse) == fin).all() and np.abs(lse[fin] - lse2[fin]).max() < 1e-12
    g = oracle.attn_bwd(q, k, v, do, sc, causal, m, L, clamp)
    g2 = oracle.attn_bwd_numpy(q, k, v, do, sc, causal, m, L, clamp)
    for a, b in zip(g, g2):
        assert np.abs(a - b).max() < 1e-12


def test_strided_views_equal_contiguous():
    B, H, S, D = 2, 3, 11, 8
    x = randn((B, S, 3, H, D), 7)             # packed [B,S,3,H,D] projection-style buffer
    q, k, v = (x[:, :, i].transpose(0, 2, 1, 3) for i in range(3))
    o1, _ = oracle.attn_fwd(q, k, v, 0.3, True)
    o2, _ = oracle.attn_fwd(np.ascontiguousarray(q), np.ascontiguousarray(k), np.ascontiguousarray(v), 0.3, True)
    assert np.array_equal(o1, o2)


def test_softmax_properties():
    B, H, S, D = 1, 2, 40, 8
    q, k = randn((B, H, S, D), 8), randn((B, H, S, D), 9)
    v = np.ones((B, H, S, D), dtype=np.float32)
    o, lse = oracle.attn_fwd(q, k, v, 0.5, True)
    assert np.abs(o - 1.0).max() < 1e-12          # rows of P sum to one
    # first causal row sees exactly one key
    s00 = 0.5 * (q[0, :, 0].astype(np.float64) * k[0, :, 0]).sum(-1)
    assert np.abs(lse[0, :, 0] - s00).max() < 1e-12


def test_backward_finite_difference():
    B, H, S, D = 1, 1, 6, 4
    q, k, v, do = (randn((B, H, S, D), s) for s in (10, 11, 12, 13))
    dq, dk, dv = oracle.attn_bwd(q, k, v, do, 0.5, True)

    def f(q_, k_, v_):
        return float((oracle.attn_fwd_numpy(q_, k_, v_, 0.5, True)[0] * do).sum())

    eps = 1e-5
    for (arr, g, idx) in ((q, dq, (0, 0, 2, 1)), (k, dk, (0, 0, 1, 3)), (v, dv, (0, 0, 4, 0))):
        hi = arr.astype(np.float64).copy(); hi[idx] += eps
        lo = arr.astype(np.float64).copy(); lo[idx] -= eps
        args_hi = [hi if a is arr else a for a in (q, k, v)]
        args_lo = [lo if a is arr else a for a in (q, k, v)]
        num = (f(*args_hi) - f(*args_lo)) / (2 * eps)
        assert abs(num - g[idx]) < 1e-7


def test_fully_hidden_rows():
    B, H, S, D = 1, 1, 4, 4
    q, k, v, do = (randn((B, H, S, D), s) for s in (14, 15, 16, 17))
    L = np.zeros(B, dtype=np.int32)
    o, lse = oracle.attn_fwd(q, k, v, 1.0, False, None, L)
    assert (o == 0).all() and np.isneginf(lse).all()
    for g in oracle.attn_bwd(q, k, v, do, 1.0, False, None, L):
        assert (g == 0).all()


@pytest.mark.parametrize("W,time_major", [(4, False), (8, True)])
def test_tsa_matches_numpy(W, time_major):
    B, S, E, H = 2, 5, 8, 2
    x = randn((B * S, E), 20)
    ws = [randn((E, H * W), 21 + i, 0.3) for i in range(3)]
    wo = randn((H * W, E), 24, 0.3)
    gamma, beta = randn((E,), 25), randn((E,), 26)
    out, y = oracle.tsa_fwd(x, *ws, wo, B, S, H, W, 1.0, time_major=time_major, gamma=gamma, beta=beta)
    X = x.astype(np.float64).reshape((S, B, E) if time_major else (B, S, E))
    if time_major:
        X = X.transpose(1, 0, 2)
    Q, K, V = [(X @ w.astype(np.float64)).reshape(B, S, H, W).transpose(0, 2, 1, 3) for w in ws]
    o, _ = oracle.attn_fwd_numpy(Q, K, V, 1.0)
    Y = o.transpose(0, 2, 1, 3).reshape(B, S, H * W) @ wo.astype(np.float64)
    Z = Y + X
    Z = (Z - Z.mean(-1, keepdims=True)) / np.sqrt(Z.var(-1, keepdims=True) + 1e-5) * gamma + beta
    if time_major:
        Z, Y = Z.transpose(1, 0, 2), Y.transpose(1, 0, 2)
    assert np.abs(Z.reshape(B * S, E) - out).max() < 1e-10
    assert np.abs(Y.reshape(B * S, E) - y).max() < 1e-12
    # backward against central differences of the fp64 forward
    dy = randn((B * S, E), 27)
    dx, dwq, dwk, dwv, dwo = oracle.tsa_bwd(x, *ws, wo, dy, B, S, H, W, 1.0, time_major=time_major)

    def F(xx, wq, wo_):
        _, yy = oracle.tsa_fwd(xx, wq, ws[1], ws[2], wo_, B, S, H, W, 1.0, time_major=time_major,
                               use_residual=False, use_layer_norm=False)
        return float((yy * dy).sum())

    eps = 1e-2
    for (name, idx, g) in (("x", (3, 2), dx), ("wq", (1, 2), dwq), ("wo", (2, 3), dwo)):
        args = dict(x=x.copy(), wq=ws[0].copy(), wo=wo.copy())
        hi = {n: a.copy() for n, a in args.items()}; hi[name][idx] += eps
        lo = {n: a.copy() for n, a in args.items()}; lo[name][idx] -= eps
        num = (F(hi["x"], hi["wq"], hi["wo"]) - F(lo["x"], lo["wq"], lo["wo"])) / (2 * eps)
        assert abs(num - g[idx]) < 2e-3 * max(1.0, abs(num))


GOLDEN = sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "ref_flash_*.npz")))


def test_golden_vectors_present():
    assert GOLDEN, "reference-generated golden vectors are missing from tests/golden/"


@pytest.mark.parametrize("path", GOLDEN, ids=[os.path.basename(p) for p in GOLDEN])
def test_oracle_matches_reference_kernel(path):
    """The golden files hold inputs and the output of the reference's own flashAttentionKernel
    (built unmodified from the reference sources, run on a B200) on its valid domain."""
    z = np.load(path)
    q, k, v, ref = z["q"], z["k"], z["v"], z["out"]
    mask = z["mask"] if "mask" in z.files else None
    o, _ = oracle.attn_fwd(q, k, v, float(z["scale"]), False, mask, None, float(z["clamp"]))
    assert np.abs(o - ref).max() < 2e-6
