"""Seeded synthetic inputs with the value distributions of the benchmark configurations.

Weights: fp32 N(0, 0.02) quantised symmetrically per output channel to int4 codes in [-7, 7]
with scale = max|w| / 7.  Activations: N(0, 1) with a fixed 0.5 % of the K channels multiplied
by 20, rounded to binary16 (and widened back to fp32 for the fp32-only entry points).  There is
no external data set on this path: every measurement and every parity case uses these.
"""
from __future__ import annotations

import numpy as np


def make_weights(K: int, N: int, seed: int = 0, std: float = 0.02):
    """fp32 N(0, std) weights quantised symmetric per output channel to int4 codes in
    [-7, 7] with scale = max|w| / 7.  Returns (B[K,N] int8 codes, w_scale[N] fp32)."""
    rng = np.random.Generator(np.random.PCG64([seed, K, N, 1]))
    W = rng.standard_normal((K, N), dtype=np.float32) * np.float32(std)
    scale = (np.abs(W).max(axis=0) / np.float32(7)).astype(np.float32)
    scale[scale == 0] = np.float32(1)
    B = np.clip(np.rint(W / scale), -7, 7).astype(np.int8)
    return B, scale


def make_activations(M: int, K: int, seed: int = 0, dtype: str = "f16"):
    """N(0,1) activations with a fixed 0.5 % of the K channels scaled by 20, rounded to
    binary16.  dtype 'f16' returns the uint16 bit patterns, 'f32' the widened values."""
    rng = np.random.Generator(np.random.PCG64([seed, M, K, 2]))
    A = rng.standard_normal((M, K), dtype=np.float32)
    n_out = max(1, int(round(0.005 * K)))
    channels = rng.choice(K, size=n_out, replace=False)
    A[:, channels] *= np.float32(20)
    h = A.astype(np.float16)
    if dtype == "f16":
        return h.view(np.uint16).copy()
    return h.astype(np.float32)


def sample_columns(N: int, count: int = 17) -> np.ndarray:
    """Evenly spaced columns, the reference's sampled check for large shapes."""
    return np.array([int(i * (N - 1) // (count - 1)) for i in range(count)], dtype=np.int32)
