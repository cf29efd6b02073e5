"""CPU oracle for pack_sequence / unpack_sequence. TEST INFRASTRUCTURE ONLY.

Restates the reference's torch path (xma/functional/sequence_packing/torch_implementation.py:9-48) with plain numpy
loops over the sequences, so that the CUDA kernels can be checked against it bit for bit. Imported by `tests/` only;
nothing that ships imports it.

Pinning: `tests/golden/sequence_packing.npz` holds outputs and gradients of the reference's own torch path on seeded
inputs (written by `tests/golden/make_golden.py`); `tests/test_oracle_golden.py` checks this file against them.
"""

from __future__ import annotations

import numpy as np


def _ranges(cu_seqlens, seq_len: int, padding_side: str):
    """-> [(b, first padded position, packed start, length)] (torch_implementation.py:13-22: with left padding the
    tokens of a sequence are its last `len` positions, with right padding its first)."""
    if padding_side not in ("left", "right"):
        raise ValueError(f"unexpected padding_side ({padding_side})")
    cu = [int(v) for v in np.asarray(cu_seqlens).reshape(-1)]
    out = []
    for b in range(len(cu) - 1):
        n = cu[b + 1] - cu[b]
        assert 0 <= n <= seq_len
        out.append((b, seq_len - n if padding_side == "left" else 0, cu[b], n))
    return out


def pack(x, cu_seqlens, padding_side: str = "left"):
    """x [B, S, ...] -> [cu_seqlens[-1], ...] (torch_implementation.py:9-26: x[batch_indices, seq_indices])."""
    x = np.asarray(x)
    total = int(np.asarray(cu_seqlens).reshape(-1)[-1])
    y = np.zeros((total, *x.shape[2:]), dtype=x.dtype)
    for b, first, start, n in _ranges(cu_seqlens, x.shape[1], padding_side):
        y[start:start + n] = x[b, first:first + n]
    return y


def unpack(x, cu_seqlens, seq_len: int, padding_side: str = "left"):
    """x [T, ...] -> [B, seq_len, ...], zeros in the padding (torch_implementation.py:29-48)."""
    x = np.asarray(x)
    batch = np.asarray(cu_seqlens).reshape(-1).shape[0] - 1
    y = np.zeros((batch, seq_len, *x.shape[1:]), dtype=x.dtype)
    for b, first, start, n in _ranges(cu_seqlens, seq_len, padding_side):
        y[b, first:first + n] = x[start:start + n]
    return y


def pack_backward(dy, cu_seqlens, seq_len: int, padding_side: str = "left"):
    """Gradient of `pack` w.r.t. x: the packed gradient put back, zeros in the padding (= unpack)."""
    return unpack(dy, cu_seqlens, seq_len, padding_side)


def unpack_backward(dy, cu_seqlens, padding_side: str = "left"):
    """Gradient of `unpack` w.r.t. x: the valid positions of the padded gradient (= pack)."""
    return pack(dy, cu_seqlens, padding_side)
