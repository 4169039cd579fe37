"""ctypes loader for the fp64 CPU oracle (TEST INFRASTRUCTURE, not product code).

Only the tests, the smoke check and the benchmark's CPU-baseline leg may import this package.
It wraps ``liboracle.so`` built from ``attn_oracle.c`` and adds a tiny numpy restatement of
the same attention contract that is used to cross-check the C code on small shapes.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liboracle.so")


def build(force: bool = False) -> str:
    """Compile liboracle.so (gcc + OpenMP) if it is missing or older than its source."""
    src = os.path.join(_HERE, "attn_oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.check_call(
            ["gcc", "-O3", "-march=x86-64-v3", "-fopenmp", "-fPIC", "-shared", "-o", _LIB_PATH, src, "-lm"]
        )
    return _LIB_PATH


class _AttnDesc(C.Structure):
    _fields_ = [
        ("B", C.c_int32), ("H", C.c_int32), ("Sq", C.c_int32), ("Sk", C.c_int32), ("D", C.c_int32),
        ("causal", C.c_int32), ("scale", C.c_float), ("score_clamp", C.c_float),
        ("q", C.c_void_p), ("q_sb", C.c_int64), ("q_sh", C.c_int64), ("q_ss", C.c_int64),
        ("k", C.c_void_p), ("k_sb", C.c_int64), ("k_sh", C.c_int64), ("k_ss", C.c_int64),
        ("v", C.c_void_p), ("v_sb", C.c_int64), ("v_sh", C.c_int64), ("v_ss", C.c_int64),
        ("keep_mask", C.c_void_p), ("kv_len", C.c_void_p),
    ]


class _TsaDesc(C.Structure):
    _fields_ = [
        ("B", C.c_int32), ("S", C.c_int32), ("E", C.c_int32), ("H", C.c_int32), ("W", C.c_int32),
        ("causal", C.c_int32), ("time_major", C.c_int32), ("use_residual", C.c_int32),
        ("use_layer_norm", C.c_int32),
        ("scale", C.c_float), ("score_clamp", C.c_float), ("ln_eps", C.c_float),
        ("x", C.c_void_p), ("wq", C.c_void_p), ("wk", C.c_void_p), ("wv", C.c_void_p), ("wo", C.c_void_p),
        ("bq", C.c_void_p), ("bk", C.c_void_p), ("bv", C.c_void_p), ("bo", C.c_void_p),
        ("gamma", C.c_void_p), ("beta", C.c_void_p),
        ("keep_mask", C.c_void_p), ("kv_len", C.c_void_p),
    ]


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        _lib = C.CDLL(_LIB_PATH)
        _lib.oracle_num_threads.restype = C.c_int
    return _lib


def num_threads() -> int:
    return int(lib().oracle_num_threads())


def set_num_threads(n: int) -> None:
    lib().oracle_set_num_threads(C.c_int(n))


def _f32(a):
    a = np.asarray(a, dtype=np.float32)
    assert a.strides[-1] == 4 or a.shape[-1] == 1, "last dimension must be contiguous"
    return a


def _ptr(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _strides3(a):
    """Element strides of (batch, head, seq) for a 4-d float32 array."""
    return [s // 4 for s in a.strides[:3]]


def _attn_desc(q, k, v, scale, causal, keep_mask, kv_len, score_clamp):
    B, H, Sq, D = q.shape
    Sk = k.shape[2]
    d = _AttnDesc()
    d.B, d.H, d.Sq, d.Sk, d.D = B, H, Sq, Sk, D
    d.causal = int(bool(causal))
    d.scale = float(scale)
    d.score_clamp = float(score_clamp) if score_clamp else 0.0
    d.q, (d.q_sb, d.q_sh, d.q_ss) = _ptr(q), _strides3(q)
    d.k, (d.k_sb, d.k_sh, d.k_ss) = _ptr(k), _strides3(k)
    d.v, (d.v_sb, d.v_sh, d.v_ss) = _ptr(v), _strides3(v)
    d.keep_mask = _ptr(keep_mask)
    d.kv_len = _ptr(kv_len)
    return d


def attn_fwd(q, k, v, scale, causal=False, keep_mask=None, kv_len=None, score_clamp=0.0,
             bh_range=None):
    """fp64 attention forward.  q [B,H,Sq,D], k/v [B,H,Sk,D] float32 (any strides with D
    contiguous).  Returns (out [B,H,Sq,D] float64, lse [B,H,Sq] float64)."""
    q, k, v = _f32(q), _f32(k), _f32(v)
    B, H, Sq, D = q.shape
    if keep_mask is not None:
        keep_mask = np.ascontiguousarray(keep_mask, dtype=np.float32)
        assert keep_mask.shape == (B, Sq, k.shape[2])
    if kv_len is not None:
        kv_len = np.ascontiguousarray(kv_len, dtype=np.int32)
    d = _attn_desc(q, k, v, scale, causal, keep_mask, kv_len, score_clamp)
    out = np.zeros((B, H, Sq, D), dtype=np.float64)
    lse = np.full((B, H, Sq), -np.inf, dtype=np.float64)
    lo, hi = bh_range if bh_range else (0, B * H)
    lib().oracle_attn_fwd(C.byref(d), _ptr(out), _ptr(lse), C.c_int(lo), C.c_int(hi))
    return out, lse


def attn_bwd(q, k, v, dout, scale, causal=False, keep_mask=None, kv_len=None, score_clamp=0.0,
             bh_range=None):
    """fp64 attention backward.  Returns (dq, dk, dv) float64, contiguous [B,H,S,D]."""
    q, k, v, dout = _f32(q), _f32(k), _f32(v), _f32(dout)
    B, H, Sq, D = q.shape
    Sk = k.shape[2]
    if keep_mask is not None:
        keep_mask = np.ascontiguousarray(keep_mask, dtype=np.float32)
    if kv_len is not None:
        kv_len = np.ascontiguousarray(kv_len, dtype=np.int32)
    d = _attn_desc(q, k, v, scale, causal, keep_mask, kv_len, score_clamp)
    dq = np.zeros((B, H, Sq, D), dtype=np.float64)
    dk = np.zeros((B, H, Sk, D), dtype=np.float64)
    dv = np.zeros((B, H, Sk, D), dtype=np.float64)
    sb, sh, ss = _strides3(dout)
    lo, hi = bh_range if bh_range else (0, B * H)
    lib().oracle_attn_bwd(C.byref(d), _ptr(dout), C.c_int64(sb), C.c_int64(sh), C.c_int64(ss),
                          _ptr(dq), _ptr(dk), _ptr(dv), C.c_int(lo), C.c_int(hi))
    return dq, dk, dv


def _tsa_desc(x, wq, wk, wv, wo, B, S, H, W, scale, causal, time_major, use_residual,
              use_layer_norm, gamma, beta, bq, bk, bv, bo, keep_mask, kv_len, score_clamp, keep):
    E = x.shape[1]
    t = _TsaDesc()
    t.B, t.S, t.E, t.H, t.W = B, S, E, H, W
    t.causal, t.time_major = int(bool(causal)), int(bool(time_major))
    t.use_residual, t.use_layer_norm = int(bool(use_residual)), int(bool(use_layer_norm))
    t.scale, t.score_clamp, t.ln_eps = float(scale), float(score_clamp or 0.0), 1e-5
    arrs = dict(x=x, wq=wq, wk=wk, wv=wv, wo=wo, bq=bq, bk=bk, bv=bv, bo=bo, gamma=gamma, beta=beta,
                keep_mask=keep_mask)
    for name, a in arrs.items():
        if a is not None:
            a = np.ascontiguousarray(a, dtype=np.float32)
            keep.append(a)
        setattr(t, name, _ptr(a))
    if kv_len is not None:
        kv_len = np.ascontiguousarray(kv_len, dtype=np.int32)
        keep.append(kv_len)
    t.kv_len = _ptr(kv_len)
    return t


def tsa_fwd(x, wq, wk, wv, wo, B, S, H, W, scale, causal=False, time_major=False,
            use_residual=True, use_layer_norm=True, gamma=None, beta=None,
            bq=None, bk=None, bv=None, bo=None, keep_mask=None, kv_len=None, score_clamp=0.0):
    """fp64 TimeSelfAttention module forward.  Returns (out [rows,E], y [rows,E]) where y is the
    projection output before residual and LayerNorm."""
    keep = []
    x = np.ascontiguousarray(x, dtype=np.float32)
    t = _tsa_desc(x, wq, wk, wv, wo, B, S, H, W, scale, causal, time_major, use_residual,
                  use_layer_norm, gamma, beta, bq, bk, bv, bo, keep_mask, kv_len, score_clamp, keep)
    out = np.zeros((B * S, x.shape[1]), dtype=np.float64)
    y = np.zeros_like(out)
    lib().oracle_tsa_fwd(C.byref(t), _ptr(out), _ptr(y))
    return out, y


def tsa_bwd(x, wq, wk, wv, wo, dy, B, S, H, W, scale, causal=False, time_major=False,
            bq=None, bk=None, bv=None, keep_mask=None, kv_len=None, score_clamp=0.0):
    """fp64 module backward.  Returns (dx, dwq, dwk, dwv, dwo)."""
    keep = []
    x = np.ascontiguousarray(x, dtype=np.float32)
    dy = np.ascontiguousarray(dy, dtype=np.float32)
    t = _tsa_desc(x, wq, wk, wv, wo, B, S, H, W, scale, causal, time_major, False, False,
                  None, None, bq, bk, bv, None, keep_mask, kv_len, score_clamp, keep)
    E, HW = x.shape[1], H * W
    dx = np.zeros((B * S, E), dtype=np.float64)
    dwq, dwk, dwv = (np.zeros((E, HW), dtype=np.float64) for _ in range(3))
    dwo = np.zeros((HW, E), dtype=np.float64)
    lib().oracle_tsa_bwd(C.byref(t), _ptr(dy), _ptr(dx), _ptr(dwq), _ptr(dwk), _ptr(dwv), _ptr(dwo))
    return dx, dwq, dwk, dwv, dwo


# ----------------------------------------------------------------------------------------------
# numpy restatement (small shapes only): an independent second statement of the same contract.
# ----------------------------------------------------------------------------------------------
def visibility(B, Sq, Sk, causal=False, keep_mask=None, kv_len=None):
    vis = np.ones((B, Sq, Sk), dtype=bool)
    if causal:
        i = np.arange(Sq)[:, None]
        j = np.arange(Sk)[None, :]
        vis &= (j <= i + (Sk - Sq))[None]
    if kv_len is not None:
        vis &= (np.arange(Sk)[None, None, :] < np.asarray(kv_len)[:, None, None])
    if keep_mask is not None:
        vis &= (np.asarray(keep_mask) != 0)
    return vis


def attn_fwd_numpy(q, k, v, scale, causal=False, keep_mask=None, kv_len=None, score_clamp=0.0):
    q, k, v = (np.asarray(a, dtype=np.float64) for a in (q, k, v))
    B, H, Sq, D = q.shape
    Sk = k.shape[2]
    s = np.einsum("bhid,bhjd->bhij", q, k) * np.float64(np.float32(scale))
    if score_clamp and score_clamp > 0:
        s = np.minimum(s, np.float64(np.float32(score_clamp)))
    vis = visibility(B, Sq, Sk, causal, keep_mask, kv_len)[:, None]
    s = np.where(vis, s, -np.inf)
    m = s.max(axis=-1, keepdims=True)
    dead = ~np.isfinite(m)
    m = np.where(dead, 0.0, m)
    p = np.exp(s - m)
    l = p.sum(axis=-1, keepdims=True)
    out = np.einsum("bhij,bhjd->bhid", p / np.where(dead, 1.0, l), v)
    lse = np.where(dead[..., 0], -np.inf, m[..., 0] + np.log(np.where(dead, 1.0, l))[..., 0])
    return out, lse


def attn_bwd_numpy(q, k, v, dout, scale, causal=False, keep_mask=None, kv_len=None, score_clamp=0.0):
    q, k, v, dout = (np.asarray(a, dtype=np.float64) for a in (q, k, v, dout))
    B, H, Sq, D = q.shape
    Sk = k.shape[2]
    sc = np.float64(np.float32(scale))
    s = np.einsum("bhid,bhjd->bhij", q, k) * sc
    clamped = np.zeros_like(s, dtype=bool)
    if score_clamp and score_clamp > 0:
        c = np.float64(np.float32(score_clamp))
        clamped = s >= c
        s = np.minimum(s, c)
    vis = visibility(B, Sq, Sk, causal, keep_mask, kv_len)[:, None]
    s = np.where(vis, s, -np.inf)
    m = s.max(axis=-1, keepdims=True)
    dead = ~np.isfinite(m)
    m = np.where(dead, 0.0, m)
    p = np.exp(s - m)
    p = p / np.where(dead, 1.0, p.sum(axis=-1, keepdims=True))
    o = np.einsum("bhij,bhjd->bhid", p, v)
    dv = np.einsum("bhij,bhid->bhjd", p, dout)
    dp = np.einsum("bhid,bhjd->bhij", dout, v)
    delta = (dout * o).sum(axis=-1, keepdims=True)
    ds = p * (dp - delta) * sc
    ds = np.where(clamped, 0.0, ds)
    dq = np.einsum("bhij,bhjd->bhid", ds, k)
    dk = np.einsum("bhij,bhid->bhjd", ds, q)
    return dq, dk, dv


# ----------------------------------------------------------------------------------------------
# FlashAttention form of the module (reference src/ml/flash_attention.cu:808-1150):
#   out = dropout( x + Wo MHA(LayerNorm(x)) + bo )
# LayerNorm on the input (:822-834, kernel :275-377, eps 1e-5, biased variance), projections with
# biases (:866-958), scores scaled by 1/sqrt(head_dim) (:998) and clamped at 10 (:167), keep-mask
# (:161-164), output projection with bias (:1075-1104), residual with the raw input (:1107-1113),
# inverted dropout last (:1117-1131).  The backward is the derivative of exactly that.
# ----------------------------------------------------------------------------------------------
def dropout_keep(seed: int, n: int, p: float) -> np.ndarray:
    """Keep decisions of n elements: the hash of (seed, index) the CUDA kernel uses (splitmix64 finaliser,
    top 24 bits as a uniform in [0, 1), keep iff u >= p)."""
    with np.errstate(over="ignore"):
        z = np.uint64(seed) + (np.arange(n, dtype=np.uint64) + np.uint64(1)) * np.uint64(0x9E3779B97F4A7C15)
        z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        z = z ^ (z >> np.uint64(31))
    u = (z >> np.uint64(40)).astype(np.float32) * np.float32(1.0 / 16777216.0)
    return u >= np.float32(p)


def layer_norm_fwd(x, gamma, beta, eps=1e-5):
    x = np.asarray(x, dtype=np.float64)
    mean = x.mean(axis=1, keepdims=True)
    inv_std = 1.0 / np.sqrt(((x - mean) ** 2).mean(axis=1, keepdims=True) + eps)
    xhat = (x - mean) * inv_std
    return xhat * np.asarray(gamma, np.float64) + np.asarray(beta, np.float64), xhat, inv_std


def layer_norm_bwd(g, xhat, inv_std, gamma):
    """(dx, dgamma, dbeta) for y = xhat * gamma + beta."""
    g = np.asarray(g, dtype=np.float64)
    gg = g * np.asarray(gamma, np.float64)
    dx = inv_std * (gg - gg.mean(axis=1, keepdims=True) - xhat * (gg * xhat).mean(axis=1, keepdims=True))
    return dx, (g * xhat).sum(axis=0), g.sum(axis=0)


def fa_fwd(x, wq, wk, wv, wo, B, S, H, D, biases=(None, None, None, None), gamma=None, beta=None,
           use_layer_norm=True, use_residual=True, keep_mask=None, dropout_prob=0.0, dropout_seed=0,
           score_clamp=10.0):
    x = np.asarray(x, dtype=np.float64)
    xin = layer_norm_fwd(x, gamma, beta)[0] if use_layer_norm else x
    bq, bk, bv, bo = biases
    _, y = tsa_fwd(xin.astype(np.float32), wq, wk, wv, wo, B, S, H, D, 1.0 / np.sqrt(D), False, False, False, False,
                   None, None, bq, bk, bv, bo, keep_mask, None, score_clamp)
    out = y + x if use_residual else y
    if dropout_prob > 0.0:
        keep = dropout_keep(dropout_seed, out.size, dropout_prob).reshape(out.shape)
        out = np.where(keep, out / (1.0 - dropout_prob), 0.0)
    return out


def fa_bwd(x, wq, wk, wv, wo, dy, B, S, H, D, biases=(None, None, None, None), gamma=None, beta=None,
           use_layer_norm=True, use_residual=True, keep_mask=None, dropout_prob=0.0, dropout_seed=0,
           score_clamp=10.0):
    """Gradients of fa_fwd.  Bias gradients come out of the weight-gradient code by giving the input a column
    of ones whose weight row is the bias."""
    x = np.asarray(x, dtype=np.float64)
    g = np.asarray(dy, dtype=np.float64)
    if dropout_prob > 0.0:
        keep = dropout_keep(dropout_seed, g.size, dropout_prob).reshape(g.shape)
        g = np.where(keep, g / (1.0 - dropout_prob), 0.0)
    E, HW = x.shape[1], H * D
    if use_layer_norm:
        xin, xhat, inv_std = layer_norm_fwd(x, gamma, beta)
    else:
        xin = x
    bq, bk, bv, _ = biases
    zeros = np.zeros(HW, np.float32)
    aug = lambda w, b: np.concatenate([np.asarray(w, np.float32), (zeros if b is None else np.asarray(b, np.float32))[None]], 0)
    x1 = np.concatenate([xin.astype(np.float32), np.ones((x.shape[0], 1), np.float32)], 1)
    wo1 = np.concatenate([np.asarray(wo, np.float32), np.zeros((HW, 1), np.float32)], 1)
    g1 = np.concatenate([g.astype(np.float32), np.zeros((x.shape[0], 1), np.float32)], 1)
    dx1, dwq1, dwk1, dwv1, dwo1 = tsa_bwd(x1, aug(wq, bq), aug(wk, bk), aug(wv, bv), wo1, g1, B, S, H, D,
                                          1.0 / np.sqrt(D), False, False, None, None, None, keep_mask, None,
                                          score_clamp)
    out = dict(dwq=dwq1[:E], dwk=dwk1[:E], dwv=dwv1[:E], dwo=dwo1[:, :E], dbq=dwq1[E], dbk=dwk1[E], dbv=dwv1[E],
               dbo=g.sum(axis=0))
    dxin = dx1[:, :E]
    if use_layer_norm:
        dx, out["dgamma"], out["dbeta"] = layer_norm_bwd(dxin, xhat, inv_std, gamma)
    else:
        dx = dxin
    out["dx"] = dx + g if use_residual else dx
    return out
