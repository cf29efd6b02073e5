"""CPU oracle for the MoE hot path. TEST INFRASTRUCTURE ONLY.

This file restates, on the CPU, the algorithm of the reference's torch path so that the CUDA
kernels can be checked against it. It is imported by `tests/`, by `__graft_entry__.smoke()` and by
`bench.py` for its CPU baseline / reference arm, and by nothing that ships: the product
(`accelerated-model-architectures_b200/`) never imports it and has no CPU path.

Integer work (histogram, stable sort, tables) is numpy; floating-point work uses torch CPU tensors
in the dtype of the inputs, rounding where the reference's torch path rounds. Every function names
the reference lines it follows (paths inside the XMA repository).

Pinning: the reference holds no golden vectors (its tests compare kernels with its own torch path on
fresh random inputs). The oracle is therefore pinned against outputs of the reference itself, run on
CPU from this repository's `tests/golden/make_golden.py`, which stores them under `tests/golden/`;
`tests/test_oracle_golden.py` checks the oracle against those files. Two rules are canonical choices
where torch leaves the result unspecified (top-k ties: lowest expert index first; sort: stable) -
for those the reference agrees on tie-free inputs and is "unpinned" on ties.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable

import numpy as np
import torch
import torch.nn.functional as F

ROW_PAD = 128


# ------------------------------------------------------------------------------------------------
# integer path
# ------------------------------------------------------------------------------------------------
def continuous_count(ids: np.ndarray, bins: int) -> np.ndarray:
    """uint32[bins] histogram; ids outside [0, bins) are ignored.
    Follows xma/functional/continuous_count/__init__.py:32-47 (`bincount(minlength=bins)`), with the
    documented "values outside the range are ignored" rule of :19-21."""
    ids = np.asarray(ids).reshape(-1)
    if bins == 1:
        return np.array([ids.size], dtype=np.uint32)
    valid = ids[(ids >= 0) & (ids < bins)]
    return np.bincount(valid.astype(np.int64), minlength=bins).astype(np.uint32)


@dataclass
class SortResult:
    counts: np.ndarray  # uint32 [E]
    offsets_incl: np.ndarray  # int32 [E]   (expert_offsets, xma/layers/moe/__init__.py:217)
    sorted_expert_idxs: np.ndarray  # int32 [R]
    sorted_scattered_idxs: np.ndarray  # int32 [R]
    pad_offsets: np.ndarray  # int32 [E+1]
    tile_prefix: np.ndarray  # int32 [E+1]
    tile_expert: np.ndarray  # int32 [tiles in use]
    row_src: np.ndarray  # int32 [padded rows in use], -1 on pad rows


def count_sort(ids: np.ndarray, num_experts: int) -> SortResult:
    """`selected_experts.flatten().sort()` + `continuous_count` + `cumsum`
    (xma/layers/moe/__init__.py:210-217) with the sort made stable (ties by flat index), plus the
    padded-layout tables the CUDA kernels derive from the counts."""
    ids = np.asarray(ids).reshape(-1).astype(np.int64)
    in_range = (ids >= 0) & (ids < num_experts)
    flat = np.nonzero(in_range)[0]
    order = flat[np.argsort(ids[flat], kind="stable")]
    counts = continuous_count(ids, num_experts) if num_experts > 1 else np.array([flat.size], dtype=np.uint32)
    offsets_incl = np.cumsum(counts.astype(np.int64)).astype(np.int32)
    tiles = (counts.astype(np.int64) + ROW_PAD - 1) // ROW_PAD
    tile_prefix = np.concatenate([[0], np.cumsum(tiles)]).astype(np.int32)
    pad_offsets = (tile_prefix.astype(np.int64) * ROW_PAD).astype(np.int32)
    tile_expert = np.repeat(np.arange(num_experts, dtype=np.int32), tiles)
    row_src = np.full(int(pad_offsets[-1]), -1, dtype=np.int32)
    start = 0
    for e in range(num_experts):
        c = int(counts[e])
        row_src[pad_offsets[e] : pad_offsets[e] + c] = order[start : start + c]
        start += c
    return SortResult(
        counts=counts,
        offsets_incl=offsets_incl,
        sorted_expert_idxs=ids[order].astype(np.int32),
        sorted_scattered_idxs=order.astype(np.int32),
        pad_offsets=pad_offsets,
        tile_prefix=tile_prefix,
        tile_expert=tile_expert,
        row_src=row_src,
    )


# ------------------------------------------------------------------------------------------------
# routing
# ------------------------------------------------------------------------------------------------
def route(logits: torch.Tensor, top_k: int) -> tuple[torch.Tensor, torch.Tensor]:
    """(router_weights [T,K] in logits.dtype, selected_experts [T,K] int64).
    Follows MoE._get_topk and the softmax of MoE._compute_routing_weights
    (xma/layers/moe/__init__.py:256-262, 192-193). Canonical tie rule: descending value, lowest
    expert index first among equal values (`sort(stable=True)`); `torch.topk` returns the same set
    of values and, on rows without ties, the same indices."""
    values, indices = torch.sort(logits.float(), dim=-1, descending=True, stable=True)
    values, indices = values[:, :top_k], indices[:, :top_k]
    weights = F.softmax(values, dim=-1).to(logits.dtype)
    return weights, indices


def route_backward(logits: torch.Tensor, selected: torch.Tensor, d_weights: torch.Tensor) -> torch.Tensor:
    """d_logits [T,E] in logits.dtype: backward of softmax (fp32) over the selected values, scattered
    to the selected columns (autograd of xma/layers/moe/__init__.py:192-193 and :260)."""
    values = torch.gather(logits.float(), 1, selected)
    w = F.softmax(values, dim=-1)
    dw = d_weights.float()
    dv = w * (dw - (w * dw).sum(-1, keepdim=True))
    d_logits = torch.zeros(logits.shape, dtype=torch.float32)
    d_logits.scatter_(1, selected, dv)
    return d_logits.to(logits.dtype)


# ------------------------------------------------------------------------------------------------
# activations
# ------------------------------------------------------------------------------------------------
def swiglu(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """xma/functional/swiglu/torch_implementation.py:9-18."""
    return (up.float() * F.silu(gate.float())).to(gate.dtype)


def swiglu_backward(gate: torch.Tensor, up: torch.Tensor, dy: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """Gradient of `up * gate * sigmoid(gate)` in fp32, rounded to the input dtype (what autograd
    gives for xma/functional/swiglu/torch_implementation.py:9-18)."""
    g, u, d = gate.float(), up.float(), dy.float()
    s = torch.sigmoid(g)
    dg = d * u * s * (1.0 + g * (1.0 - s))
    du = d * g * s
    return dg.to(gate.dtype), du.to(gate.dtype)


def swiglu_packed(x: torch.Tensor) -> torch.Tensor:
    """xma/functional/swiglu/torch_implementation.py:21-30 (gate = even, up = odd features)."""
    xf = x.float()
    return (xf[..., 1::2] * F.silu(xf[..., ::2])).to(x.dtype)


def swiglu_packed_backward(x: torch.Tensor, dy: torch.Tensor) -> torch.Tensor:
    dg, du = swiglu_backward(x[..., ::2], x[..., 1::2], dy)
    dx = torch.empty_like(x)
    dx[..., ::2] = dg
    dx[..., 1::2] = du
    return dx


def _act_swiglu_chunk(h: torch.Tensor) -> torch.Tensor:
    g, u = h.chunk(2, dim=-1)
    return swiglu(g, u)


def _act_swiglu_chunk_bwd(h: torch.Tensor, da: torch.Tensor) -> torch.Tensor:
    g, u = h.chunk(2, dim=-1)
    dg, du = swiglu_backward(g, u, da)
    return torch.cat([dg, du], dim=-1)


def _act_glu(h: torch.Tensor) -> torch.Tensor:
    return F.glu(h, dim=-1)


def _act_glu_bwd(h: torch.Tensor, da: torch.Tensor) -> torch.Tensor:
    a, b = h.float().chunk(2, dim=-1)
    s = torch.sigmoid(b)
    d = da.float()
    return torch.cat([d * s, d * a * s * (1 - s)], dim=-1).to(h.dtype)


def _act_gelu_tanh(h: torch.Tensor) -> torch.Tensor:
    return F.gelu(h, approximate="tanh")


def _act_gelu_tanh_bwd(h: torch.Tensor, da: torch.Tensor) -> torch.Tensor:
    x = h.float()
    k = 0.7978845608028654
    inner = k * (x + 0.044715 * x**3)
    t = torch.tanh(inner)
    dt = (1 - t * t) * k * (1 + 3 * 0.044715 * x * x)
    return (da.float() * (0.5 * (1 + t) + 0.5 * x * dt)).to(h.dtype)


ACTIVATIONS: dict[str, tuple[Callable, Callable]] = {
    "swiglu": (_act_swiglu_chunk, _act_swiglu_chunk_bwd),
    "swiglu_packed": (swiglu_packed, swiglu_packed_backward),
    "glu": (_act_glu, _act_glu_bwd),
    "gelu_tanh": (_act_gelu_tanh, _act_gelu_tanh_bwd),
}


# ------------------------------------------------------------------------------------------------
# the layer
# ------------------------------------------------------------------------------------------------
@dataclass
class MoEResult:
    y: torch.Tensor
    router_logits: torch.Tensor
    router_weights: torch.Tensor
    selected_experts: torch.Tensor
    sort: SortResult
    grads: dict = field(default_factory=dict)  # "x", "gate", "c_fc", "c_proj", "router_weights"


def moe_forward_backward(
    x: torch.Tensor,
    gate_w: torch.Tensor,
    w1: torch.Tensor,
    w2: torch.Tensor,
    top_k: int,
    activation: str = "swiglu",
    dy: torch.Tensor | None = None,
    router_logits: torch.Tensor | None = None,
) -> MoEResult:
    """Forward (and, when `dy` is given, backward) of the reference's torch path:
    MoE.forward / _compute_routing_weights / _compute_experts torch branch and Experts.torch_forward
    (xma/layers/moe/__init__.py:162-195, 235-250, 89-105). All tensors are CPU tensors of one dtype;
    `router_logits` may be supplied to take the gate projection's rounding out of a comparison.

    x [T,H], gate_w [E,H], w1 [E,N1,H], w2 [E,H,I]. The backward is written out by hand."""
    T, H = x.shape
    E = gate_w.shape[0]
    act, act_bwd = ACTIVATIONS[activation]
    dtype = x.dtype

    logits = F.linear(x, gate_w) if router_logits is None else router_logits
    weights, selected = route(logits, top_k)
    srt = count_sort(selected.numpy(), E)
    perm = torch.from_numpy(srt.sorted_scattered_idxs.astype(np.int64))
    fan_in = perm // top_k
    gates = weights.flatten()[perm]
    freq = [int(c) for c in srt.counts]

    xs = x[fan_in]
    xs_e = list(xs.split(freq, dim=0))
    h_e = [F.linear(xs_e[e], w1[e]) for e in range(E)]
    a_e = [act(h) for h in h_e]
    o_e = [F.linear(a_e[e], w2[e]) for e in range(E)]
    o = torch.cat(o_e, dim=0)
    scaled = o * gates.unsqueeze(-1)
    y = torch.zeros((T, H), dtype=dtype).index_add(0, fan_in, scaled)

    res = MoEResult(y=y, router_logits=logits, router_weights=weights, selected_experts=selected, sort=srt)
    if dy is None:
        return res

    do = dy[fan_in]
    d_gates = (do.float() * o.float()).sum(-1).to(dtype)
    d_o = (do * gates.unsqueeze(-1)).split(freq, dim=0)
    d_w1 = torch.zeros_like(w1)
    d_w2 = torch.zeros_like(w2)
    d_xs = []
    for e in range(E):
        if freq[e] == 0:
            d_xs.append(torch.zeros((0, H), dtype=dtype))
            continue
        d_a = d_o[e] @ w2[e]
        d_w2[e] = d_o[e].t() @ a_e[e]
        d_h = act_bwd(h_e[e], d_a)
        d_w1[e] = d_h.t() @ xs_e[e]
        d_xs.append(d_h @ w1[e])
    d_xs = torch.cat(d_xs, dim=0)
    d_x = torch.zeros((T, H), dtype=dtype).index_add(0, fan_in, d_xs)

    d_weights = torch.zeros(T * top_k, dtype=dtype)
    d_weights[perm] = d_gates
    d_weights = d_weights.view(T, top_k)
    d_logits = route_backward(logits, selected, d_weights)
    res.grads = {
        "router_weights": d_weights,
        "router_logits": d_logits,
        "c_fc": d_w1,
        "c_proj": d_w2,
        "x_experts": d_x,
    }
    if router_logits is None:
        res.grads["gate"] = d_logits.t() @ x
        res.grads["x"] = d_x + d_logits @ gate_w
    return res


def expert_weight_grads_slice(
    xs_e: torch.Tensor,
    d_o_e: torch.Tensor,
    w1_e: torch.Tensor,
    w2_e: torch.Tensor,
    cols: torch.Tensor,
) -> tuple[torch.Tensor, torch.Tensor]:
    """Weight gradients of ONE SwiGLU expert restricted to the intermediate features `cols`
    (gate = first half of c_fc's outputs, up = second half), so that the check of a large expert
    costs a fraction of its full backward. Same arithmetic as the per-expert loop of
    `moe_forward_backward` (xma/layers/moe/__init__.py:89-105 forward, autograd backward), in fp32:

      xs_e  [rows, H]   the token rows routed to the expert (expert-sorted order)
      d_o_e [rows, H]   dY of those rows already multiplied by their routing weight
      w1_e  [2I, H], w2_e [H, I]
      returns d_w1[cols and I + cols, :]  as [2 * len(cols), H]  and  d_w2[:, cols]  as [H, len(cols)]
    """
    inter = w2_e.shape[1]
    xs, do = xs_e.float(), d_o_e.float()
    gate = xs @ w1_e[cols].float().t()
    up = xs @ w1_e[cols + inter].float().t()
    # the kernels keep gate|up in the storage dtype and apply SwiGLU to the rounded values
    gate, up = gate.to(xs_e.dtype), up.to(xs_e.dtype)
    act = swiglu(gate, up)
    d_w2 = do.t() @ act.float()
    d_act = do @ w2_e[:, cols].float()
    dg, du = swiglu_backward(gate.float(), up.float(), d_act)
    d_w1 = torch.cat([dg.t() @ xs, du.t() @ xs], dim=0)
    return d_w1, d_w2
