"""CPU restatement of the reference's RMSNorm.  TEST INFRASTRUCTURE ONLY: imported by tests/ and the
benchmark's CPU-baseline leg; the product never calls it.

Follows reference norm.rs in f32 numpy: `inverse_rms` (:124-127), `forward` (:41-62), `backward` (:69-121)
with its tiles of 32 rows whose partial weight gradients are added in order (:8-14, :113-117).
Pinned by the reference's own five tests (norm.rs:138-216: unit RMS, no mean subtraction, per-channel
weight, both finite-difference checks with the reference's inputs and tolerances); see
tests/test_rmsnorm_oracle.py.
"""
from __future__ import annotations

import numpy as np

F = np.float32
ROWS_PER_TILE = 32


def inverse_rms(x: np.ndarray, eps: float) -> np.ndarray:
    x = x.astype(F)
    mean_square = (x * x).sum(axis=1, dtype=F) / F(x.shape[1])
    return (F(1.0) / np.sqrt(mean_square + F(eps))).astype(F)


def forward(x: np.ndarray, weight: np.ndarray, eps: float) -> np.ndarray:
    x = x.astype(F)
    return (x * inverse_rms(x, eps)[:, None] * weight.astype(F)[None, :]).astype(F)


def backward(x: np.ndarray, weight: np.ndarray, grad_y: np.ndarray, eps: float, grad_weight: np.ndarray = None):
    """Returns (grad_x, grad_weight); `grad_weight` (optional) is the gradient accumulated so far."""
    x, g, w = x.astype(F), grad_y.astype(F), weight.astype(F)
    rows, d = x.shape
    inv = inverse_rms(x, eps)
    projection = (g * w[None, :] * x).sum(axis=1, dtype=F)
    shared = (projection * inv * inv * inv / F(d)).astype(F)
    grad_x = (g * w[None, :] * inv[:, None] - x * shared[:, None]).astype(F)
    gw = np.zeros(d, F) if grad_weight is None else grad_weight.astype(F).copy()
    contrib = (g * x * inv[:, None]).astype(F)
    for t0 in range(0, rows, ROWS_PER_TILE):
        partial = np.zeros(d, F)
        for r in range(t0, min(rows, t0 + ROWS_PER_TILE)):   # rows of a tile in order
            partial = (partial + contrib[r]).astype(F)
        gw = (gw + partial).astype(F)                        # tiles in order
    return grad_x, gw
