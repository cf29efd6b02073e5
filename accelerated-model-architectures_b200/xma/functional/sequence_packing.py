"""`pack_sequence` / `unpack_sequence`: between a padded batch `[B, S, ...]` and its packed form `[T, ...]` (the valid
tokens of sequence 0, then of sequence 1, ...), given the cumulative sequence lengths. Same calls as the reference's
(xma/functional/sequence_packing/__init__.py:39-132); each direction is one CUDA kernel that copies every sequence as
one contiguous byte range (csrc/sequence_packing.cu), and unpacking writes the zero padding in the same pass.
The backward of either is the other direction on the gradient (cuda_implementation.py:137-212)."""

from __future__ import annotations

from typing import Sequence

import torch

from .. import ops
from .._lib import require_cuda
from ..accelerator import KernelBackend


class _PackSequence(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x: torch.Tensor, cu_seqlens: torch.Tensor, output_shape: tuple, left: bool) -> torch.Tensor:
        x = x.contiguous()
        ctx.save_for_backward(cu_seqlens)
        ctx.left, ctx.x_shape = left, x.shape
        y = torch.empty(output_shape, device=x.device, dtype=x.dtype)
        ops.pack_sequence_(x, cu_seqlens, y, left)
        return y

    @staticmethod
    def backward(ctx, dy: torch.Tensor):
        (cu_seqlens,) = ctx.saved_tensors
        dx = torch.empty(ctx.x_shape, device=dy.device, dtype=dy.dtype)  # the kernel writes the zeros too
        ops.unpack_sequence_(dy.contiguous(), cu_seqlens, dx, ctx.left)
        return dx, None, None, None


class _UnpackSequence(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x: torch.Tensor, cu_seqlens: torch.Tensor, output_shape: tuple, left: bool) -> torch.Tensor:
        x = x.contiguous()
        ctx.save_for_backward(cu_seqlens)
        ctx.left, ctx.x_shape = left, x.shape
        y = torch.empty(output_shape, device=x.device, dtype=x.dtype)
        ops.unpack_sequence_(x, cu_seqlens, y, left)
        return y

    @staticmethod
    def backward(ctx, dy: torch.Tensor):
        (cu_seqlens,) = ctx.saved_tensors
        # (rows beyond cu_seqlens[-1], which the forward never read, get their zero gradient from the kernel)
        dx = torch.empty(ctx.x_shape, device=dy.device, dtype=dy.dtype)
        ops.pack_sequence_(dy.contiguous(), cu_seqlens, dx, ctx.left)
        return dx, None, None, None


def _check(kernel_backend, padding_side: str, inputs) -> bool:
    if kernel_backend not in (None, KernelBackend.cuda):
        raise ValueError(f"unexpected kernel_backend ({kernel_backend})")
    assert padding_side in ["left", "right"]
    assert isinstance(inputs, (list, tuple))
    return padding_side == "left"


def pack_sequence(
    inputs: Sequence[torch.Tensor],
    cu_seqlens: torch.Tensor,
    total_tokens: int,
    padding_side: str = "left",
    *,
    kernel_backend: KernelBackend | None = None,
) -> Sequence[torch.Tensor]:
    """Every `x` of `inputs` is `[B, S, ...]`; returns the list of `[total_tokens, ...]` tensors in which row
    `cu_seqlens[b] + i` is token `i` of sequence `b` (its last `len_b` positions with `padding_side="left"`, its
    first with `"right"`). `cu_seqlens` is `[B + 1]`, int32 / uint32 / int64, on the device."""
    left = _check(kernel_backend, padding_side, inputs)
    cu_seqlens = cu_seqlens.contiguous()
    outputs = []
    for x in inputs:
        assert x.dim() >= 2
        assert x.size(0) == cu_seqlens.size(0) - 1
        require_cuda(x, cu_seqlens)
        outputs.append(_PackSequence.apply(x, cu_seqlens, (total_tokens, *x.size()[2:]), left))
    return outputs


def unpack_sequence(
    inputs: Sequence[torch.Tensor],
    cu_seqlens: torch.Tensor,
    batch_size: int,
    sequence_length: int,
    padding_side: str = "left",
    *,
    kernel_backend: KernelBackend | None = None,
) -> Sequence[torch.Tensor]:
    """Every `x` of `inputs` is `[T, ...]`; returns the list of `[batch_size, sequence_length, ...]` tensors with the
    tokens of sequence `b` in row `b` and zeros in the padding."""
    left = _check(kernel_backend, padding_side, inputs)
    cu_seqlens = cu_seqlens.contiguous()
    outputs = []
    for x in inputs:
        assert x.dim() >= 2
        assert cu_seqlens.size(0) - 1 == batch_size
        require_cuda(x, cu_seqlens)
        outputs.append(_UnpackSequence.apply(x, cu_seqlens, (batch_size, sequence_length, *x.size()[1:]), left))
    return outputs
