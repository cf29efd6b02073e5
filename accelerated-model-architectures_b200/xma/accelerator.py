"""`KernelBackend` / `Accelerator` enums with the member names of the reference
(xma/accelerator.py:22-170), kept so that `kernel_backend=` arguments written for the reference keep
working. There is exactly one implementation behind them here: the sm_100a CUDA kernels. `None` and
`KernelBackend.cuda` select it; every other value is rejected by the entry points (no dispatch, no
CPU fallback).
"""

from __future__ import annotations

from enum import Enum

import torch


class KernelBackend(Enum):
    cuda = "cuda"
    jax = "jax"
    mps = "mps"
    nki = "nki"
    pallas = "pallas"
    rocm = "rocm"
    torch = "torch"
    triton = "triton"

    def get_compatible_accelerator(self) -> "Accelerator":
        found = Accelerator.get_accelerator()
        if self == KernelBackend.torch:
            return found
        return Accelerator.cuda if self == KernelBackend.cuda else None

    def verify_accelerator(self) -> bool:
        return self.get_compatible_accelerator() == Accelerator.get_accelerator()


class Accelerator(Enum):
    cpu = "cpu"
    cuda = "cuda"
    mps = "mps"
    rocm = "rocm"
    tpu = "tpu"
    trainium = "trainium"

    @staticmethod
    def get_accelerator() -> "Accelerator":
        return Accelerator.cuda if torch.cuda.is_available() else Accelerator.cpu

    @staticmethod
    def get_current_device() -> int | str:
        return torch.cuda.current_device() if torch.cuda.is_available() else "cpu"

    @staticmethod
    def device_count() -> int:
        return torch.cuda.device_count() if torch.cuda.is_available() else 1

    @staticmethod
    def get_kernel_backend() -> KernelBackend:
        return KernelBackend.cuda

    @staticmethod
    def synchronize() -> None:
        if torch.cuda.is_available():
            torch.cuda.synchronize()

    @staticmethod
    def get_core_count() -> int:
        return torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count


def resolve_kernel_backend(kernel_backend: KernelBackend | None) -> KernelBackend:
    """The only accepted values are None and KernelBackend.cuda; anything else raises ValueError,
    the exception the reference raises for a backend an op does not have
    (xma/functional/continuous_count/__init__.py:48-49, xma/layers/moe/__init__.py:251-252)."""
    if kernel_backend is None or kernel_backend == KernelBackend.cuda:
        return KernelBackend.cuda
    raise ValueError(f"unexpected kernel_backend ({kernel_backend})")
