"""Seeded inputs and error measures shared by the tests."""
from __future__ import annotations

import numpy as np


def randn(shape, seed, scale=1.0):
    return (np.random.default_rng(seed).standard_normal(shape) * scale).astype(np.float32)


def bf16_round(a: np.ndarray) -> np.ndarray:
    """float32 -> nearest-even bfloat16 -> float32, in numpy."""
    a = np.ascontiguousarray(a, dtype=np.float32)
    u = a.view(np.uint32).astype(np.uint64)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16
    return r.astype(np.uint32).view(np.float32)


def max_abs(a, b) -> float:
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    return float(np.max(np.abs(a - b))) if a.size else 0.0


def rel_l2(a, ref) -> float:
    a = np.asarray(a, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    den = float(np.sqrt(np.sum(ref * ref)))
    return float(np.sqrt(np.sum((a - ref) ** 2))) / (den if den > 0 else 1.0)


def keep_mask(B, Sq, Sk, seed, p_keep=0.7, dead_rows=((0, 0),)):
    """Dense float keep-mask (0 hides).  `dead_rows` lists (batch, query) rows hidden entirely."""
    m = (np.random.default_rng(seed).random((B, Sq, Sk)) < p_keep).astype(np.float32)
    for b, i in dead_rows:
        if b < B and i < Sq:
            m[b, i, :] = 0.0
    return m


def std_uniform_stream(seed: int, n: int, lo: float, hi: float) -> np.ndarray:
    """The first `n` draws of ``std::uniform_real_distribution<float>(lo, hi)`` fed by ``std::mt19937(seed)``
    (libstdc++): one 32-bit output per draw, u = float(raw) * 2^-32 (clamped just below 1), value = u * (hi - lo)
    + lo in float arithmetic.  ``numpy.random.RandomState(seed)`` seeds MT19937 the way std::mt19937 does."""
    raw = np.random.RandomState(seed)._bit_generator.random_raw(n).astype(np.float32)
    u = (raw * np.float32(2.0 ** -32)).astype(np.float32)
    u = np.where(u >= 1, np.nextafter(np.float32(1), np.float32(0)), u).astype(np.float32)
    lo32, hi32 = np.float32(lo), np.float32(hi)
    return (u * (hi32 - lo32) + lo32).astype(np.float32)


def reference_tsa_weight_blob(E: int, H: int, seed: int) -> np.ndarray:
    """Payload of the weight file the reference's cuDNN TimeSelfAttention writes for (input_dim E, H heads, seed):
    Wq, Wk, Wv, Wo drawn in that order from one generator, each with limit sqrt(6 / (E + E))
    (reference src/ml/cuDNN_ops.cu:34-96; every head is E wide, include/cuDNN_ops.h:166-169)."""
    lim = np.sqrt(np.float32(6.0) / np.float32(E + E)).astype(np.float32)
    return std_uniform_stream(seed, 4 * E * H * E, -lim, lim)
