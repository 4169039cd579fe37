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
