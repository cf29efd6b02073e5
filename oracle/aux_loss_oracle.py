"""CPU oracle for the auxiliary load-balancing loss. TEST INFRASTRUCTURE ONLY.

PARITY UNPINNED: the reference has no load-balancing loss (it returns `router_logits` unused,
xma/layers/moe/__init__.py:180), so there are no outputs of the reference to pin this file against. It restates the
published definition (Switch Transformer, Fedus et al. 2021, eq. 4-6, in the form used with top-k routing):

    p = softmax(logits),  P_e = mean_t p[t, e],  f_e = (slots routed to e) / tokens,  loss = E * sum_e f_e * P_e

in float64 numpy, with the top-k rule of the layer's own oracle (descending value, lowest expert index first among
equals: xma/layers/moe/__init__.py:256-262 made canonical), and its analytic gradient. The tests also check it against
torch autograd of the same formula. Imported by `tests/` only.
"""

from __future__ import annotations

import numpy as np


def select(logits: np.ndarray, top_k: int) -> np.ndarray:
    """[T, K] expert ids: stable descending sort, first k."""
    order = np.argsort(-logits.astype(np.float64), axis=-1, kind="stable")
    return order[:, :top_k]


def loss(logits: np.ndarray, top_k: int) -> tuple[float, np.ndarray]:
    """-> (loss, f [E])."""
    x = logits.astype(np.float64)
    T, E = x.shape
    p = np.exp(x - x.max(axis=-1, keepdims=True))
    p /= p.sum(axis=-1, keepdims=True)
    f = np.bincount(select(logits, top_k).reshape(-1), minlength=E).astype(np.float64) / T
    return float(E * (f * p.mean(axis=0)).sum()), f


def grad(logits: np.ndarray, top_k: int, d_loss: float = 1.0) -> np.ndarray:
    """d loss / d logits [T, E] (f carries no gradient): p * (c - sum_e c_e p_e), c = d_loss * E * f / T."""
    x = logits.astype(np.float64)
    T, E = x.shape
    p = np.exp(x - x.max(axis=-1, keepdims=True))
    p /= p.sum(axis=-1, keepdims=True)
    _, f = loss(logits, top_k)
    c = d_loss * E * f / T
    return p * (c[None, :] - (p * c[None, :]).sum(axis=-1, keepdims=True))
