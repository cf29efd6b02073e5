"""`fused_residual_add_rmsnorm`: the residual add + RMSNorm that sits in front of the MoE layer in a transformer
block. Same call as the reference's (xma/functional/fused_residual_add_rmsnorm/__init__.py:27-83); one CUDA
kernel forward, one backward (csrc/rmsnorm.cu)."""

from __future__ import annotations

import torch

from .. import ops
from .._lib import require_cuda
from ..accelerator import KernelBackend


# Rows of the weight-gradient partial sums = CTAs of the backward kernel: 4 per SM of a B200 (148 SMs). A constant, so
# that nothing but tensor allocations and the opaque custom ops sit in the traced backward.
_DW_PARTIAL_ROWS = 592


def _eps(eps: float | None, dtype: torch.dtype) -> float:
    return float(torch.finfo(dtype).eps if eps is None else eps)  # template.py:20-21, 58-59


class _FusedResidualAddRMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, residual, weight, eps, multiplier, memory_efficient):
        needs_grad = any(ctx.needs_input_grad[:3])
        m = 1.0 if multiplier is None else float(multiplier)
        y = torch.empty_like(x, memory_format=torch.contiguous_format)
        # the value the norm sees is an output when a residual comes in; without one it equals x unless a
        # multiplier applies, in which case the backward needs its own copy of x * multiplier
        keep_scaled = residual is None and m != 1.0 and needs_grad
        xr = torch.empty_like(x, memory_format=torch.contiguous_format) if residual is not None or keep_scaled else None
        rstd = (torch.empty(x.size(0), device=x.device, dtype=torch.float32)
                if needs_grad and not memory_efficient else None)
        ops.rmsnorm_fwd_(x, residual, weight, y, xr, rstd, _eps(eps, x.dtype), m)
        if needs_grad:
            ctx.save_for_backward(x if xr is None else xr, weight, rstd)
        ctx.eps, ctx.multiplier, ctx.has_residual = _eps(eps, x.dtype), m, residual is not None
        ctx.set_materialize_grads(False)
        if residual is None:
            return y, None
        return y, xr

    @staticmethod
    def backward(ctx, dy, dxr):
        xr, weight, rstd = ctx.saved_tensors
        if dy is None:
            dy = torch.zeros_like(xr)
        if dy.stride(-1) != 1:
            dy = dy.contiguous()
        if dxr is not None and dxr.stride(-1) != 1:
            dxr = dxr.contiguous()
        dx = torch.empty_like(xr)
        dr = torch.empty_like(xr) if ctx.has_residual else None
        dw_partial = None
        if weight is not None and ctx.needs_input_grad[2]:
            blocks = min(max(xr.size(0), 1), _DW_PARTIAL_ROWS)
            dw_partial = torch.empty(blocks, xr.size(1), device=xr.device, dtype=torch.float32)
        ops.rmsnorm_bwd_(xr, weight, dy, dxr, rstd, dx, dr, dw_partial, ctx.eps, ctx.multiplier)
        dw = None if dw_partial is None else dw_partial.sum(0).to(weight.dtype)
        return dx, dr, dw, None, None, None


def fused_residual_add_rmsnorm(
    x: torch.Tensor,
    residual: torch.Tensor | None,
    weight: torch.Tensor | None,
    eps: float | None,
    multiplier: float | None = None,
    memory_efficient: bool = False,
    *,
    kernel_backend: KernelBackend | None = None,
) -> tuple[torch.Tensor, torch.Tensor | None]:
    """`y = rms_norm(x * multiplier + residual) * weight`; returns `(y, updated residual stream)` (the second is
    None without a residual). `memory_efficient=False` keeps the row-wise 1/rms for the backward; True recomputes it.

    Deviation from the reference, on a case its tests do not reach: with a multiplier and no residual the reference
    saves the unscaled `x` for the backward (triton_implementation/__init__.py:37), so its gradient is that of
    `rms_norm(x) * multiplier`; here the backward differentiates what the forward computed."""
    if kernel_backend not in (None, KernelBackend.cuda):
        raise ValueError(f"unexpected kernel_backend ({kernel_backend})")
    if x.dim() != 2:
        raise AssertionError("x should be 2D")
    if residual is not None:
        assert residual.dim() == 2 and residual.size() == x.size()
        assert residual.dtype == x.dtype, "tensors residual and x should have same dtype"
    if weight is not None:
        assert weight.dim() == 1, "weight should be 1D"
        assert weight.size(-1) == x.size(-1), "hidden size for x and weight tensor is different"
        assert weight.dtype == x.dtype, "tensors weight and y should have same dtype"
        weight = weight.contiguous()
    require_cuda(x, residual, weight)
    if x.size(1) > 1 and x.stride(1) != 1:
        x = x.contiguous()
    if residual is not None and residual.size(1) > 1 and residual.stride(1) != 1:
        residual = residual.contiguous()
    return _FusedResidualAddRMSNorm.apply(x, residual, weight, eps, multiplier, memory_efficient)
