"""CPU oracle for fused_residual_add_rmsnorm. TEST INFRASTRUCTURE ONLY.

Restates the reference's torch path (xma/functional/fused_residual_add_rmsnorm/torch_implementation.py:9-27:
optional `x * multiplier`, optional `+ residual`, `F.rms_norm`) and writes its backward out by hand, in float64
numpy, so that the CUDA kernels can be checked against it. Imported by `tests/` only; nothing that ships imports it.

Pinning: `tests/golden/rmsnorm.npz` holds outputs and gradients of the reference's own torch path on seeded inputs
(written by `tests/golden/make_golden.py`); `tests/test_oracle_golden.py` checks this file against them.
"""

from __future__ import annotations

import numpy as np


def forward(x, residual, weight, eps: float, multiplier):
    """-> (y, xr or None, rstd). torch_implementation.py:17-25; `F.rms_norm` = v * rsqrt(mean(v^2) + eps) * W."""
    v = np.asarray(x, dtype=np.float64)
    if multiplier not in (None, 1):
        v = v * float(multiplier)
    xr = None
    if residual is not None:
        v = v + np.asarray(residual, dtype=np.float64)
        xr = v
    rstd = 1.0 / np.sqrt((v * v).mean(axis=-1, keepdims=True) + eps)
    y = v * rstd
    if weight is not None:
        y = y * np.asarray(weight, dtype=np.float64)
    return y, xr, rstd


def backward(x, residual, weight, eps: float, multiplier, dy, dxr):
    """-> (dx, dresidual or None, dweight or None) for upstream gradients dy (of y) and dxr (of the updated
    residual stream; None when it is unused). With z = v * rstd and g = dy * W:
    dv = (g - z * mean(g * z)) * rstd + dxr, dresidual = dv, dx = dv * multiplier, dW = sum_rows dy * z."""
    m = 1.0 if multiplier in (None, 1) else float(multiplier)
    v = np.asarray(x, dtype=np.float64) * m
    if residual is not None:
        v = v + np.asarray(residual, dtype=np.float64)
    rstd = 1.0 / np.sqrt((v * v).mean(axis=-1, keepdims=True) + eps)
    z = v * rstd
    dy = np.asarray(dy, dtype=np.float64)
    g = dy if weight is None else dy * np.asarray(weight, dtype=np.float64)
    dv = (g - z * (g * z).mean(axis=-1, keepdims=True)) * rstd
    if dxr is not None:
        dv = dv + np.asarray(dxr, dtype=np.float64)
    dw = None if weight is None else (dy * z).sum(axis=0)
    return dv * m, (dv if residual is not None else None), dw
