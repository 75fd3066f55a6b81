"""Seeded synthetic inputs for the five benchmark configurations. TEST INFRASTRUCTURE - see
oracle/__init__.py. Everything is drawn on the host with np.random.default_rng(seed) (PCG64) in
float32, in the order written here, so the device kernels, the NumPy baseline and the reference's own
CUDA ops all see identical bits. No dataset is involved: shapes and distributions only."""
from __future__ import annotations

from typing import Dict, Sequence

import numpy as np

__all__ = ["mlp_params", "mlp_batch", "gemm_inputs", "softmax_inputs", "ce_inputs", "adam_inputs"]


def mlp_params(dims: Sequence[int], seed: int) -> Dict[str, np.ndarray]:
    """He-normal weights (OUT, IN) ~ N(0, sqrt(2/IN)), zero biases; names '<2i>.W', '<2i>.b'."""
    rng = np.random.default_rng(seed)
    out: Dict[str, np.ndarray] = {}
    for i in range(len(dims) - 1):
        out[f"{2 * i}.W"] = (rng.standard_normal((dims[i + 1], dims[i]), dtype=np.float32) * np.float32(np.sqrt(2.0 / dims[i])))
        out[f"{2 * i}.b"] = np.zeros((dims[i + 1],), np.float32)
    return out


def mlp_batch(batch: int, in_dim: int, classes: int, seed: int):
    """X ~ N(0,1) float32 [batch, in_dim]; labels uniform int32 in [0, classes). Drawn after the
    parameters from an independent stream (seed + 1000) so parameter and data draws do not interleave."""
    rng = np.random.default_rng(seed + 1000)
    x = rng.standard_normal((batch, in_dim), dtype=np.float32)
    y = rng.integers(0, classes, size=(batch,), dtype=np.int32)
    return x, y


def gemm_inputs(M: int, N: int, K: int, seed: int = 1):
    """A [M,K], B [K,N] ~ U(-1,1) float32 (round to bf16 for the bf16 case), bias ~ N(0,1) [N]."""
    rng = np.random.default_rng(seed)
    A = rng.uniform(-1.0, 1.0, size=(M, K)).astype(np.float32)
    B = rng.uniform(-1.0, 1.0, size=(K, N)).astype(np.float32)
    bias = rng.standard_normal((N,), dtype=np.float32)
    return A, B, bias


def softmax_inputs(M: int, N: int, seed: int = 2):
    """X ~ N(0, 3) (sigma = 3) float32 [M, N]."""
    return np.random.default_rng(seed).standard_normal((M, N), dtype=np.float32) * np.float32(3.0)


def ce_inputs(B: int, Cn: int, seed: int = 2):
    """logits ~ N(0, 2) (sigma = 2) float32 [B, C]; labels uniform int32 in [0, C)."""
    rng = np.random.default_rng(seed + 1)
    z = rng.standard_normal((B, Cn), dtype=np.float32) * np.float32(2.0)
    y = rng.integers(0, Cn, size=(B,), dtype=np.int32)
    return z, y


def adam_inputs(n: int, seed: int = 3):
    """p ~ N(0, 0.02), g ~ N(0, 1e-3), float32 [n]; m = v = 0."""
    rng = np.random.default_rng(seed)
    p = rng.standard_normal((n,), dtype=np.float32) * np.float32(0.02)
    g = rng.standard_normal((n,), dtype=np.float32) * np.float32(1e-3)
    return p, g
