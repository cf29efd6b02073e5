"""`continuous_count` with the signature and return type of the reference
(xma/functional/continuous_count/__init__.py:15-51), running the sm_100a histogram kernel."""

from __future__ import annotations

import torch

from ..accelerator import KernelBackend, resolve_kernel_backend
from ..ops import continuous_count_


@torch.no_grad()
def continuous_count(x: torch.Tensor, bins: int, *, kernel_backend: KernelBackend | None = None) -> torch.Tensor:
    """Counts the occurrences of the values [0, 1, ..., `bins`) in `x` (`bins` excluded). Values
    outside that range are ignored (and flagged in the device status word).

    :param x: 1-D int32 or int64 CUDA tensor
    :param bins: number of counters
    :param kernel_backend: None or KernelBackend.cuda; anything else raises ValueError
    :return: uint32 tensor of shape [bins]
    """

    if bins == 1:
        return torch.tensor([x.numel()], dtype=torch.uint32, device=x.device)

    assert x.dim() == 1, "x should be 1-dimensional"
    assert x.dtype in [torch.int32, torch.long]

    resolve_kernel_backend(kernel_backend)
    if not x.is_cuda:
        raise RuntimeError("xma.functional.continuous_count (B200 build) needs CUDA tensors; there is no CPU path")

    if not x.is_contiguous():
        x = x.contiguous()

    y = torch.empty(bins, dtype=torch.int32, device=x.device)
    continuous_count_(x, y)
    return y.view(torch.uint32)
