"""Comparison helpers shared by the GPU parity tests."""

from __future__ import annotations

import random

import numpy as np
import torch

# Outputs and gradients must lie within max rel err 2e-2 of an fp32 reference for bf16 (4e-3 fp16, 2e-4 fp32).
REL_TOL = {torch.float32: 2e-4, torch.float16: 4e-3, torch.bfloat16: 2e-2}


def max_rel_err(got: torch.Tensor, ref: torch.Tensor) -> float:
    """max |got - ref| / max |ref| (error normalised by the tensor's scale)."""
    got = got.detach().double().cpu()
    ref = ref.detach().double().cpu()
    scale = max(float(ref.abs().max()), 1e-30)
    return float((got - ref).abs().max()) / scale


def assert_close_rel(got: torch.Tensor, ref: torch.Tensor, tol: float, what: str = "") -> None:
    assert got.shape == ref.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(ref.shape)}"
    assert torch.isfinite(got.float()).all(), f"{what}: non-finite values"
    err = max_rel_err(got, ref)
    assert err <= tol, f"{what}: max rel err {err:.3e} > {tol:.1e}"


def sizes_1d(log_max_power_of_2: int = 15, max_offset: int = 10, num_not_powers_of_2: int = 50) -> list[int]:
    """The size list of the reference's tests (tests/utils.py:17-28): 2^i + j and 50 sizes in 2000..4000."""
    rng = random.Random(0)
    sizes = set()
    for i in range(log_max_power_of_2):
        for j in range(max_offset):
            sizes.add(2**i + j)
    for _ in range(num_not_powers_of_2):
        sizes.add(3000 + rng.randint(-1000, 1000))
    return sorted(sizes)


def zipf_ids(n: int, bins: int, s: float, seed: int) -> np.ndarray:
    """Zipf(s)-distributed bin ids by inverse-CDF sampling of ranks, ranks shuffled over bins."""
    rng = np.random.RandomState(seed)
    p = 1.0 / np.arange(1, bins + 1) ** s
    cdf = np.cumsum(p / p.sum())
    ranks = np.searchsorted(cdf, rng.random_sample(n), side="right").clip(0, bins - 1)
    perm = rng.permutation(bins)
    return perm[ranks].astype(np.int32)
