"""Seeded input generators shared by `make_golden.py` (which runs the reference on them) and by the
tests (which run the oracle and the CUDA kernels on the same values). numpy's Mersenne-Twister
streams are stable across versions and machines, unlike torch's device RNG."""

from __future__ import annotations

import numpy as np
import torch

# name -> (tokens, hidden, intermediate, experts, top_k, activation)
MOE_CASES = {
    "tiny_swiglu": (48, 32, 48, 4, 2, "swiglu"),
    "tiny_glu": (40, 32, 24, 6, 2, "glu"),
    "tiny_gelu": (33, 24, 40, 5, 3, "gelu_tanh"),
    "tiny_packed": (37, 32, 16, 4, 2, "swiglu_packed"),
    "empty_experts": (7, 64, 32, 16, 2, "swiglu"),
    # the CPU-runnable layer: tokens=512, hidden=256, intermediate=512, 8 experts, top-2, fp32, seed 0
    "config1": (512, 256, 512, 8, 2, "swiglu"),
}

COUNT_CASES = {"n1": (1, 72), "n33": (33, 72), "n1024_e8": (1024, 8), "n4099": (4099, 72), "n70000_e256": (70000, 256)}

SWIGLU_CASES = {"s17x24": (17, 24), "s64x128": (64, 128), "s5x3": (5, 3)}

# name -> (rows, cols, residual, weight, multiplier)
RMSNORM_CASES = {
    "r9x7": (9, 7, True, True, 0.9),
    "r33x64": (33, 64, True, True, None),
    "r12x100_noweight": (12, 100, True, False, 0.9),
    "r8x256_noresidual": (8, 256, False, True, None),
    "r5x3000": (5, 3000, True, True, 0.9),
}
RMSNORM_EPS = 1e-5

# pack_sequence / unpack_sequence: name -> (cumulative sequence lengths, padded length S, trailing shape).
# The first is the reference test's own cu_seqlens (tests/functional/pack_sequence_test.py:28) at a reduced S.
PACK_CASES = {
    "ref_cu_3x4": ([0, 70, 170, 295, 393, 412, 515, 691], 180, (3, 4)),
    "ragged_9x7": ([0, 5, 5, 17, 18, 40], 23, (9, 7)),
    "scalar_rows": ([0, 3, 11, 12], 9, (1, 1)),
    "full_and_empty": ([0, 6, 6, 12], 6, (3,)),
}


def moe_inputs(name: str, dtype: torch.dtype = torch.float32, seed: int = 0):
    """x ~ N(0,1); gate and expert weights ~ N(0, 0.02); dy ~ N(0,1). Values are rounded to `dtype`
    first, so the fp32 oracle and a bf16 kernel see exactly the same numbers."""
    T, H, I, E, K, act = MOE_CASES[name]
    rng = np.random.RandomState(seed)
    n1 = I if act == "gelu_tanh" else 2 * I

    def t(a):
        return torch.from_numpy(a.astype(np.float32)).to(dtype)

    x = t(rng.standard_normal((T, H)))
    gate = t(rng.standard_normal((E, H)) * 0.02)
    w1 = t(rng.standard_normal((E, n1, H)) * 0.02)
    w2 = t(rng.standard_normal((E, H, I)) * 0.02)
    dy = t(rng.standard_normal((T, H)))
    return dict(x=x, gate=gate, w1=w1, w2=w2, dy=dy, top_k=K, activation=act, num_experts=E)


def count_inputs(name: str, seed: int = 42) -> tuple[np.ndarray, int]:
    n, bins = COUNT_CASES[name]
    rng = np.random.RandomState(seed)
    return rng.randint(0, bins, size=n).astype(np.int64), bins


def swiglu_inputs(name: str, seed: int = 7):
    """Integer-valued inputs in [-8, 8), the distribution the reference's swiglu tests use
    (tests/utils.py:49-63)."""
    rows, cols = SWIGLU_CASES[name]
    rng = np.random.RandomState(seed)
    g = torch.from_numpy(rng.randint(-8, 8, size=(rows, cols)).astype(np.float32))
    u = torch.from_numpy(rng.randint(-8, 8, size=(rows, cols)).astype(np.float32))
    return g, u


def rmsnorm_inputs(name: str, seed: int = 11):
    """x, residual ~ N(0,1); weight ~ N(1, 0.1); upstream gradients of both outputs ~ N(0,1)."""
    rows, cols, has_r, has_w, multiplier = RMSNORM_CASES[name]
    rng = np.random.RandomState(seed)
    f = lambda a: torch.from_numpy(a.astype(np.float32))
    x = f(rng.standard_normal((rows, cols)))
    r = f(rng.standard_normal((rows, cols))) if has_r else None
    w = f(1.0 + 0.1 * rng.standard_normal(cols)) if has_w else None
    dy = f(rng.standard_normal((rows, cols)))
    dxr = f(rng.standard_normal((rows, cols))) if has_r else None
    return dict(x=x, residual=r, weight=w, dy=dy, dxr=dxr, multiplier=multiplier)


def pack_inputs(name: str, seed: int = 0):
    """Padded batch x [B, S, ...] and packed batch p [T, ...] of fp32 N(0,1) values, with upstream gradients for the
    packed (`dpacked`) and the padded (`dpadded`) results."""
    cu, S, trailing = PACK_CASES[name]
    rng = np.random.RandomState(seed)
    f = lambda *s: torch.from_numpy(rng.standard_normal(s).astype(np.float32))
    B, T = len(cu) - 1, cu[-1]
    return dict(cu_seqlens=cu, seq_len=S, x=f(B, S, *trailing), p=f(T, *trailing), dpacked=f(T, *trailing),
                dpadded=f(B, S, *trailing))


def sample(t: torch.Tensor, limit: int = 4096) -> np.ndarray:
    """Evenly strided subsample of a tensor (all of it when small), as float32/int64 numpy."""
    flat = t.detach().reshape(-1)
    if flat.numel() > limit:
        step = flat.numel() // limit
        flat = flat[::step][:limit]
    return flat.to(torch.float32).numpy() if flat.is_floating_point() else flat.to(torch.int64).numpy()
