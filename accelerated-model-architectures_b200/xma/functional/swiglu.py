"""`swiglu` / `swiglu_packed` with the signatures of the reference
(xma/functional/swiglu/__init__.py:39-87), forward and backward on the sm_100a kernels."""

from __future__ import annotations

import torch

from ..accelerator import KernelBackend, resolve_kernel_backend
from ..ops import swiglu_bwd_, swiglu_fwd_, swiglu_packed_bwd_, swiglu_packed_fwd_


def _rows(t: torch.Tensor) -> torch.Tensor:
    """2-D view whose last dimension is contiguous (row-strided views such as the halves of
    `chunk(2, -1)` are passed through without a copy)."""
    if t.dim() == 2 and (t.size(1) <= 1 or t.stride(1) == 1):
        return t
    return t.contiguous()


def _as_rows(t: torch.Tensor) -> torch.Tensor:
    """Any shape the elementwise reference accepts -> [rows, last dimension] (0-D and 1-D become one row)."""
    if t.dim() == 2:
        return t
    if t.dim() < 2:
        return t.reshape(1, -1)
    return t.flatten(0, -2)


class _Swiglu(torch.autograd.Function):
    @staticmethod
    def forward(ctx, g: torch.Tensor, u: torch.Tensor) -> torch.Tensor:
        g, u = _rows(g), _rows(u)
        if any(ctx.needs_input_grad):
            ctx.save_for_backward(g, u)
        y = torch.empty(g.shape, dtype=g.dtype, device=g.device)
        swiglu_fwd_(g, u, y)
        return y

    @staticmethod
    def backward(ctx, dy: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        g, u = ctx.saved_tensors
        dy = _rows(dy)
        dg = torch.empty(g.shape, dtype=g.dtype, device=g.device)
        du = torch.empty(u.shape, dtype=u.dtype, device=u.device)
        swiglu_bwd_(g, u, dy, dg, du)
        return dg, du


class _SwigluPacked(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x: torch.Tensor) -> torch.Tensor:
        x = _rows(x)
        if any(ctx.needs_input_grad):
            ctx.save_for_backward(x)
        y = torch.empty(x.size(0), x.size(1) // 2, dtype=x.dtype, device=x.device)
        swiglu_packed_fwd_(x, y)
        return y

    @staticmethod
    def backward(ctx, dy: torch.Tensor) -> torch.Tensor:
        (x,) = ctx.saved_tensors
        dy = _rows(dy)
        dx = torch.empty(x.shape, dtype=x.dtype, device=x.device)
        swiglu_packed_bwd_(x, dy, dx)
        return dx


def swiglu(gate: torch.Tensor, up: torch.Tensor, *, kernel_backend: KernelBackend | None = None) -> torch.Tensor:
    """computes swiglu activation as `up * gate * sigmoid(gate)`

    :param gate: `gate` activation tensor
    :param up: `up` activation tensor
    :param kernel_backend: None or KernelBackend.cuda
    :return: output tensor
    """

    assert gate.size() == up.size(), "tensors gate and up should have same shape"
    assert gate.type() == up.type(), "tensors gate and up should have same dtype"
    resolve_kernel_backend(kernel_backend)
    if not gate.is_cuda:
        raise RuntimeError("xma.functional.swiglu (B200 build) needs CUDA tensors; there is no CPU path")

    original_shape = gate.size()
    gate, up = _as_rows(gate), _as_rows(up)

    y = _Swiglu.apply(gate, up)
    return y.view(original_shape)


def swiglu_packed(x: torch.Tensor, *, kernel_backend: KernelBackend | None = None) -> torch.Tensor:
    """computes swiglu activation by splitting the tensor `x` into 2 parts: gate and up activations. The tensor has
    interleaved values of gate, up, gate, up, ...

    :param x: input activation
    :param kernel_backend: None or KernelBackend.cuda
    :return: output tensor
    """

    resolve_kernel_backend(kernel_backend)
    if not x.is_cuda:
        raise RuntimeError("xma.functional.swiglu_packed (B200 build) needs CUDA tensors; there is no CPU path")
    original_shape = x.size()
    if original_shape[-1] % 2 != 0:
        raise ValueError(f"{original_shape[-1]} is not divisible by 2")
    x = _as_rows(x)

    y = _SwigluPacked.apply(x)
    return y.view(*original_shape[:-1], original_shape[-1] // 2)


def swiglu_chunked(x: torch.Tensor, *, kernel_backend: KernelBackend | None = None) -> torch.Tensor:
    """`swiglu(*x.chunk(2, dim=-1))`: gate = first half of the last dimension, up = second half. The usual way to
    give `xma.layers.MoE` a SwiGLU activation; unlike a lambda around `swiglu`, the layer can recognise this
    function (and `swiglu_packed`) by the tag below and fuse it into its GEMM epilogues."""
    gate, up = x.chunk(2, dim=-1)
    return swiglu(gate, up, kernel_backend=kernel_backend)


# `MoE` fuses an activation_function that carries one of these tags (a plain attribute, so user code can tag
# its own equivalent callable): "swiglu" = gate | up halves, "swiglu_packed" = gate, up interleaved.
swiglu_chunked.xma_fused_activation = "swiglu"
swiglu_packed.xma_fused_activation = "swiglu_packed"
