"""`MoE` / `Experts` with the constructor, parameters and forward signature of the reference
(xma/layers/moe/__init__.py:22-262), computed by the sm_100a kernels of libxma_b200.so.

Data flow of one forward (R = tokens * top_k routed rows):
  gate projection (torch / cuBLAS) -> route_topk_softmax -> count_sort (counts, offsets, stable
  permutation, padded row map, tile tables) -> gather_rows (token rows -> padded grouped rows)
  -> grouped GEMM up (+ fused SwiGLU) -> [activation] -> grouped GEMM down, rows scattered to
  flat (token, slot) order -> combine_rows with the routing weights.
Backward mirrors xma/layers/moe/triton_implementation/__init__.py:41-72 and :110-162, except that the
down projection is not recomputed (its unweighted output is kept for d_router_weights).
"""

from __future__ import annotations

import os
import warnings
from dataclasses import dataclass
from typing import Callable

import torch
import torch.nn as nn

from ... import ops
from ..._lib import (EPI_DSWIGLU, EPI_DSWIGLU_PACKED, EPI_PLAIN, EPI_SWIGLU, EPI_SWIGLU_PACKED, IMPL_SIMT, ROW_PAD,
                     W_KN, W_NK, dtype_code, lib, raise_on_device_status)
from ...accelerator import KernelBackend, resolve_kernel_backend
from ...functional import swiglu, swiglu_packed


class SwiGLU(nn.Module):
    """`swiglu(*x.chunk(2, dim=-1))`: gate = first half of the features, up = second half. Passing an
    instance as `activation_function` (with `is_glu=True`) lets `MoE` fuse the activation into the
    epilogue of the up-projection GEMM; called on its own it runs the stand-alone kernel."""

    xma_fused_activation = "swiglu"

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        gate, up = x.chunk(2, dim=-1)
        return swiglu(gate, up)


class SwiGLUPacked(nn.Module):
    """`swiglu_packed(x)`: gate/up interleaved along the feature dimension."""

    xma_fused_activation = "swiglu_packed"

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return swiglu_packed(x)


@dataclass
class RoutePlan:
    """Everything the expert kernels need to know about one routing decision (all int32, on device)."""

    num_experts: int
    top_k: int
    num_rows: int  # R = tokens * top_k
    tile_cap: int  # allocated 128-row tiles: R // 128 + E
    counts: torch.Tensor  # [E]   rows per expert (int32 storage, same bits as the reference's uint32)
    offsets_incl: torch.Tensor  # [E]   inclusive prefix sum (expert_offsets of the reference)
    pad_offsets: torch.Tensor  # [E+1] first padded grouped row of each expert
    tile_prefix: torch.Tensor  # [E+1] tiles in front of each expert, [E] = tiles in use
    tile_expert: torch.Tensor  # [tile_cap]
    sorted_expert_idxs: torch.Tensor  # [R]
    sorted_scattered_idxs: torch.Tensor  # [R]
    row_src: torch.Tensor  # [tile_cap * 128] flat index of each padded grouped row, -1 = pad
    row_dst: torch.Tensor = None  # [R] the inverse: padded grouped row of each flat index

    @property
    def row_cap(self) -> int:
        return self.tile_cap * ROW_PAD

    @property
    def rows_in_use(self) -> torch.Tensor:
        return self.pad_offsets[self.num_experts :]

    @property
    def expert_frequency(self) -> torch.Tensor:
        return self.counts.view(torch.uint32)


@torch.no_grad()
def build_route_plan(selected_experts: torch.Tensor, num_experts: int) -> RoutePlan:
    """Stable counting sort of the routed expert ids; replaces `.flatten().sort()`, `continuous_count`
    and `cumsum` of xma/layers/moe/__init__.py:210-217."""
    tokens, top_k = selected_experts.shape
    ids = selected_experts.reshape(-1)
    R = ids.numel()
    dev = ids.device
    tile_cap = R // ROW_PAD + num_experts
    i32 = dict(dtype=torch.int32, device=dev)
    plan = RoutePlan(
        num_experts=num_experts,
        top_k=top_k,
        num_rows=R,
        tile_cap=tile_cap,
        counts=torch.empty(num_experts, **i32),
        offsets_incl=torch.empty(num_experts, **i32),
        pad_offsets=torch.empty(num_experts + 1, **i32),
        tile_prefix=torch.empty(num_experts + 1, **i32),
        tile_expert=torch.empty(tile_cap, **i32),
        sorted_expert_idxs=torch.empty(R, **i32),
        sorted_scattered_idxs=torch.empty(R, **i32),
        row_src=torch.empty(tile_cap * ROW_PAD, **i32),
        row_dst=torch.empty(R, **i32),
    )
    ops.count_sort_(
        ids, num_experts, plan.counts, plan.offsets_incl, plan.pad_offsets, plan.tile_prefix, plan.tile_expert,
        plan.sorted_expert_idxs, plan.sorted_scattered_idxs, plan.row_src, plan.row_dst,
    )
    return plan


class _TopKSoftmax(torch.autograd.Function):
    """router_logits [T, E] -> (router_weights [T, K] in the logits dtype, selected_experts [T, K] int32)."""

    @staticmethod
    def forward(ctx, logits: torch.Tensor, top_k: int):
        logits = logits if logits.stride(-1) == 1 else logits.contiguous()
        T = logits.size(0)
        weights = torch.empty(T, top_k, dtype=logits.dtype, device=logits.device)
        selected = torch.empty(T, top_k, dtype=torch.int32, device=logits.device)
        ops.route_topk_softmax_(logits, top_k, weights, selected)
        ctx.save_for_backward(logits, selected)
        ctx.mark_non_differentiable(selected)
        return weights, selected

    @staticmethod
    def backward(ctx, d_weights: torch.Tensor, _d_selected):
        logits, selected = ctx.saved_tensors
        d_logits = torch.empty(logits.shape, dtype=logits.dtype, device=logits.device)
        ops.route_topk_softmax_bwd_(logits, selected, d_weights.contiguous(), d_logits)
        return d_logits, None


def _plan_tensors(plan: RoutePlan):
    return (plan.counts, plan.pad_offsets, plan.tile_prefix, plan.tile_expert, plan.row_src)


class _UpProjectionExperts(torch.autograd.Function):
    """x [T, H] -> expert-sorted, padded rows [row_cap, N] = x[token of row] @ W_e^T
    (xma/layers/moe/triton_implementation/__init__.py:12-72)."""

    @staticmethod
    def forward(ctx, x, weight, top_k, counts, pad_offsets, tile_prefix, tile_expert, row_src):
        E, N, H = weight.shape
        row_cap = row_src.numel()
        xs = torch.empty(row_cap, H, dtype=x.dtype, device=x.device)
        ops.gather_rows_(x, row_src, None, top_k, pad_offsets[E:], xs)
        out = torch.zeros(row_cap, N, dtype=x.dtype, device=x.device)
        ops.grouped_gemm_rows_(xs, weight, W_NK, out, None, None, tile_expert, tile_prefix, H, N, EPI_PLAIN,
                               ops.GEMM_IMPL)
        ctx.save_for_backward(xs, weight, counts, pad_offsets, tile_prefix, tile_expert, row_src)
        ctx.top_k = top_k
        ctx.tokens = x.size(0)
        return out

    @staticmethod
    def backward(ctx, grad_out):
        xs, weight, counts, pad_offsets, tile_prefix, tile_expert, row_src = ctx.saved_tensors
        E, N, H = weight.shape
        grad_out = grad_out.contiguous()
        d_weight = d_input = None
        if ctx.needs_input_grad[1]:
            d_weight = torch.empty_like(weight)
            ops.grouped_gemm_dw_(grad_out, xs, counts, pad_offsets, d_weight, ops.GEMM_IMPL)
        if ctx.needs_input_grad[0]:
            R = ctx.tokens * ctx.top_k
            dxs = torch.empty(R, H, dtype=xs.dtype, device=xs.device)
            ops.grouped_gemm_rows_(grad_out, weight, W_KN, dxs, None, row_src, tile_expert, tile_prefix, N, H,
                                   EPI_PLAIN, ops.GEMM_IMPL)
            d_input = torch.empty(ctx.tokens, H, dtype=xs.dtype, device=xs.device)
            ops.combine_rows_(dxs, None, ctx.top_k, d_input)
        return d_input, d_weight, None, None, None, None, None, None


class _DownProjectionExperts(torch.autograd.Function):
    """grouped rows [row_cap, I] -> y [T, H] = sum_k w[t, k] * (row(t, k) @ W_e^T)
    (xma/layers/moe/triton_implementation/__init__.py:75-162)."""

    @staticmethod
    def forward(ctx, h, weight, router_weights, counts, pad_offsets, tile_prefix, tile_expert, row_src):
        E, H, I = weight.shape
        T, K = router_weights.shape
        h = h.contiguous()
        ys = torch.empty(T * K, H, dtype=h.dtype, device=h.device)
        ops.grouped_gemm_rows_(h, weight, W_NK, ys, None, row_src, tile_expert, tile_prefix, I, H, EPI_PLAIN,
                               ops.GEMM_IMPL)
        y = torch.empty(T, H, dtype=h.dtype, device=h.device)
        router_weights = router_weights.contiguous()
        ops.combine_rows_(ys, router_weights, K, y)
        ctx.save_for_backward(h, weight, router_weights, ys, counts, pad_offsets, tile_prefix, tile_expert, row_src)
        return y

    @staticmethod
    def backward(ctx, grad_out):
        h, weight, router_weights, ys, counts, pad_offsets, tile_prefix, tile_expert, row_src = ctx.saved_tensors
        E, H, I = weight.shape
        T, K = router_weights.shape
        grad_out = grad_out.contiguous()
        d_router_weights = None
        if ctx.needs_input_grad[2]:
            d_router_weights = torch.empty_like(router_weights)
            ops.combine_bwd_(ys, grad_out, K, d_router_weights)
        dys = torch.empty(row_src.numel(), H, dtype=h.dtype, device=h.device)
        ops.gather_rows_(grad_out, row_src, router_weights.view(-1), K, pad_offsets[E:], dys)
        d_weight = d_input = None
        if ctx.needs_input_grad[1]:
            d_weight = torch.empty_like(weight)
            ops.grouped_gemm_dw_(dys, h, counts, pad_offsets, d_weight, ops.GEMM_IMPL)
        if ctx.needs_input_grad[0]:
            d_input = torch.zeros(row_src.numel(), I, dtype=h.dtype, device=h.device)
            ops.grouped_gemm_rows_(dys, weight, W_KN, d_input, None, None, tile_expert, tile_prefix, H, I,
                                   EPI_PLAIN, ops.GEMM_IMPL)
        return d_input, d_weight, d_router_weights, None, None, None, None, None


class _FusedSwiGLUExperts(torch.autograd.Function):
    """Whole expert block with SwiGLU fused into the GEMM epilogues:
    y[t] = sum_k w[t,k] * (swiglu(x[t] @ W1_e^T) @ W2_e^T), e = selected_experts[t, k].
    With `router_weights=None` every row of x is one routed row (top_k = 1) and the unweighted expert
    output is returned in the order of x (the expert-parallel layer combines on the home rank)."""

    @staticmethod
    def forward(ctx, x, w1, w2, router_weights, counts, pad_offsets, tile_prefix, tile_expert, row_src,
                packed=False, row_dst=None):
        E, two_i, H = w1.shape
        I = two_i // 2
        ctx.packed = packed
        weighted = router_weights is not None
        T, K = router_weights.shape if weighted else (x.size(0), 1)
        row_cap = row_src.numel()
        opts = dict(dtype=x.dtype, device=x.device)
        impl = ops.GEMM_IMPL

        xs = torch.empty(row_cap, H, **opts)
        if row_dst is not None:
            # token-major: every token row is read once and written to the rows of its K slots
            ops.spread_rows_(x, row_dst, None, None, None, K, counts, pad_offsets, xs)
        else:
            ops.gather_rows_(x, row_src, None, K, pad_offsets[E:], xs)
        gu = torch.empty(row_cap, two_i, **opts)
        act = torch.empty(row_cap, I, **opts)
        ops.grouped_gemm_rows_(xs, w1, W_NK, act, gu, None, tile_expert, tile_prefix, H, two_i,
                               EPI_SWIGLU_PACKED if packed else EPI_SWIGLU, impl, tag="gemm_up_swiglu")
        ys = torch.empty(T * K, H, **opts)
        ops.grouped_gemm_rows_(act, w2, W_NK, ys, None, row_src, tile_expert, tile_prefix, I, H, EPI_PLAIN, impl,
                               tag="gemm_down")
        if weighted:
            router_weights = router_weights.contiguous()
            y = torch.empty(T, H, **opts)
            ops.combine_rows_(ys, router_weights, K, y)
            ctx.save_for_backward(xs, gu, act, ys, w1, w2, router_weights, counts, pad_offsets, tile_prefix,
                                  tile_expert, row_src)
        else:
            y = ys
            ctx.save_for_backward(xs, gu, act, w1, w2, counts, pad_offsets, tile_prefix, tile_expert, row_src)
        ctx.weighted = weighted
        ctx.tokens, ctx.top_k = T, K
        ctx.row_dst = row_dst
        return y

    @staticmethod
    def backward(ctx, grad_out):
        if ctx.weighted:
            (xs, gu, act, ys, w1, w2, router_weights, counts, pad_offsets, tile_prefix, tile_expert,
             row_src) = ctx.saved_tensors
        else:
            xs, gu, act, w1, w2, counts, pad_offsets, tile_prefix, tile_expert, row_src = ctx.saved_tensors
            ys = router_weights = None
        E, two_i, H = w1.shape
        I = two_i // 2
        T, K = ctx.tokens, ctx.top_k
        row_cap = row_src.numel()
        opts = dict(dtype=xs.dtype, device=xs.device)
        impl = ops.GEMM_IMPL
        grad_out = grad_out.contiguous()
        need_x, need_w1, need_w2, need_rw = ctx.needs_input_grad[:4]

        d_rw = None
        dys = torch.empty(row_cap, H, **opts)
        coeff = router_weights.view(-1) if ctx.weighted else None
        if ctx.row_dst is not None:
            # one pass: dY[t] is read once, scaled into its K grouped rows, and dotted with the K expert outputs
            if need_rw and ctx.weighted:
                d_rw = torch.empty_like(router_weights)
                ops.spread_rows_(grad_out, ctx.row_dst, coeff, ys, d_rw, K, counts, pad_offsets, dys)
            else:
                ops.spread_rows_(grad_out, ctx.row_dst, coeff, None, None, K, counts, pad_offsets, dys)
        else:
            if need_rw and ctx.weighted:
                d_rw = torch.empty_like(router_weights)
                ops.combine_bwd_(ys, grad_out, K, d_rw)
            ops.gather_rows_(grad_out, row_src, coeff, K, pad_offsets[E:], dys)

        d_w2 = None
        if need_w2:
            d_w2 = torch.empty_like(w2)
            ops.grouped_gemm_dw_(dys, act, counts, pad_offsets, d_w2, impl, tag="gemm_dw2")

        d_x = d_w1 = None
        if need_x or need_w1:
            dgu = torch.empty(row_cap, two_i, **opts)
            ops.grouped_gemm_rows_(dys, w2, W_KN, dgu, gu, None, tile_expert, tile_prefix, H, I,
                                   EPI_DSWIGLU_PACKED if ctx.packed else EPI_DSWIGLU, impl, tag="gemm_dact_dswiglu")
            if need_w1:
                d_w1 = torch.empty_like(w1)
                ops.grouped_gemm_dw_(dgu, xs, counts, pad_offsets, d_w1, impl, tag="gemm_dw1")
            if need_x:
                dxs = torch.empty(T * K, H, **opts)
                ops.grouped_gemm_rows_(dgu, w1, W_KN, dxs, None, row_src, tile_expert, tile_prefix, two_i, H,
                                       EPI_PLAIN, impl, tag="gemm_dx")
                if K == 1:
                    d_x = dxs
                else:
                    d_x = torch.empty(T, H, **opts)
                    ops.combine_rows_(dxs, None, K, d_x)
        return d_x, d_w1, d_w2, d_rw, None, None, None, None, None, None, None


# XMA_B200_CHECK_STATUS=1: `MoE.forward` reads the device status word after every call (one host synchronisation)
_CHECK_STATUS = os.environ.get("XMA_B200_CHECK_STATUS", "0") not in ("", "0")


class Experts(nn.Module):
    """Per-expert linear weights `[num_experts, out_features, in_features]`; same parameters and
    buffers as the reference (xma/layers/moe/__init__.py:22-43, 112-119) so state dicts interchange."""

    def __init__(
        self, num_experts: int, in_features: int, out_features: int, add_bias: bool = True, std: float | None = None
    ) -> None:
        super().__init__()
        self.weight = nn.Parameter(torch.empty(num_experts, out_features, in_features))
        self.bias = None
        if add_bias:
            self.bias = nn.Parameter(torch.empty(num_experts, out_features))
        self.std = std
        self.num_experts = num_experts
        self.in_features = in_features
        self.out_features = out_features
        self.register_buffer("N_array", torch.empty((num_experts,), dtype=torch.uint32))
        self.register_buffer("K_array", torch.empty((num_experts,), dtype=torch.uint32))
        self.reset_parameters()

    def extra_repr(self) -> str:
        return "num_experts={}, in_features={}, out_features={}".format(
            self.num_experts, self.in_features, self.out_features
        )

    @torch.no_grad()
    def reset_parameters(self) -> None:
        nn.init.normal_(self.weight, mean=0, std=self.std)
        if self.bias is not None:
            self.bias.zero_()
        self.N_array.fill_(self.out_features)
        self.K_array.fill_(self.in_features)


class MoE(nn.Module):
    def __init__(
        self,
        num_experts: int,
        num_experts_per_tok: int,
        hidden_size: int,
        intermediate_size: int,
        activation_function: Callable,
        is_glu: bool,
        add_bias: bool,
        std: float,
    ) -> None:
        super().__init__()
        self.num_experts = num_experts
        self.top_k = num_experts_per_tok
        self.hidden_size = hidden_size
        self.intermediate_size = intermediate_size

        self.gate = nn.Linear(in_features=self.hidden_size, out_features=num_experts, bias=False)
        self.c_fc = Experts(
            num_experts=num_experts,
            in_features=self.hidden_size,
            out_features=2 * self.intermediate_size if is_glu else self.intermediate_size,
            add_bias=add_bias,
            std=std,
        )
        self.act = activation_function
        self.c_proj = Experts(
            num_experts=num_experts,
            in_features=self.intermediate_size,
            out_features=self.hidden_size,
            add_bias=add_bias,
            std=std,
        )
        self.is_glu = is_glu
        self._probed = False

    def forward(self, x: torch.Tensor, *, kernel_backend: KernelBackend | None = None) -> tuple[torch.Tensor, torch.Tensor]:
        resolve_kernel_backend(kernel_backend)
        if not x.is_cuda:
            raise RuntimeError("xma.layers.MoE (B200 build) needs CUDA tensors; there is no CPU path")
        original_shape = x.shape
        x = x.reshape(-1, self.hidden_size)

        router_logits, router_weights, selected_experts = self._compute_routing_weights(x)
        x = self._compute_experts(x, router_weights, selected_experts)
        x = x.view(original_shape)
        if _CHECK_STATUS and not torch.compiler.is_compiling():
            raise_on_device_status(x.device)  # synchronises; off by default (see xma.check_device_status)
        return x, router_logits

    def _fused_activation(self, x: torch.Tensor) -> str | None:
        """"swiglu" / "swiglu_packed" when the activation is one the GEMM epilogues implement: recognised by its
        `xma_fused_activation` tag (`xma.layers.SwiGLU`, `SwiGLUPacked`, `xma.functional.swiglu_chunked`,
        `swiglu_packed`). An untagged callable (a lambda around `swiglu`, say) cannot be recognised by looking
        at it; the first eager call evaluates it on 4 x 16 probe values and warns if it computes SwiGLU, because
        it then runs as GEMM -> stand-alone kernel -> GEMM instead of the fused path."""
        if not self.is_glu:
            return None
        tag = getattr(self.act, "xma_fused_activation", None)
        if tag in ("swiglu", "swiglu_packed"):
            return tag
        if not self._probed and not torch.compiler.is_compiling():
            self._probed = True
            try:
                with torch.no_grad():
                    probe = torch.linspace(-3.0, 3.0, 64, device=x.device, dtype=torch.float32).view(4, 16)
                    got = self.act(probe)
                    for name, fn in (("swiglu_chunked", lambda h: swiglu(*h.chunk(2, dim=-1))),
                                     ("swiglu_packed", swiglu_packed)):
                        if got.shape == (4, 8) and torch.allclose(got, fn(probe), rtol=1e-5, atol=1e-6):
                            warnings.warn(
                                f"xma.layers.MoE: activation_function computes SwiGLU but is not tagged, so it runs "
                                f"unfused; pass xma.functional.{name} (or xma.layers.SwiGLU / SwiGLUPacked, or set "
                                f"`.xma_fused_activation` on the callable) to fuse it into the grouped GEMMs",
                                stacklevel=3)
            except Exception:  # an activation that rejects the probe is simply not SwiGLU
                pass
        return None

    def _compute_routing_weights(self, x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        # x -> (total_q, hidden_size)
        router_logits = self.gate(x)
        # router_logits -> (total_q, num_experts)
        router_weights, selected_experts = _TopKSoftmax.apply(router_logits, self.top_k)
        # router_weights -> (total_q, top_k) in x.dtype, selected_experts -> (total_q, top_k) int32
        return router_logits, router_weights, selected_experts

    def _tensor_cores(self, x: torch.Tensor) -> bool:
        """True when the grouped GEMMs of this layer run on the tcgen05 kernels."""
        if ops.GEMM_IMPL == IMPL_SIMT:
            return False
        code = dtype_code(x.dtype)
        return bool(lib.xma_b200_grouped_gemm_uses_tensor_cores(code, self.hidden_size, self.intermediate_size)) \
            and self.intermediate_size % 8 == 0

    def _compute_experts(
        self, x: torch.Tensor, router_weights: torch.Tensor, selected_experts: torch.Tensor
    ) -> torch.Tensor:
        # the kernel path of the reference has no bias support either (xma/layers/moe/__init__.py:53,75)
        assert self.c_fc.bias is None and self.c_proj.bias is None, "expert biases are not supported"
        if x.size(0) == 0:
            # nothing is routed: an empty result that still hands exact zero gradients to every parameter
            zero = (self.c_fc.weight.sum() + self.c_proj.weight.sum() + router_weights.sum()) * 0
            return x + zero.to(x.dtype)
        x = x.contiguous()
        plan = build_route_plan(selected_experts, self.num_experts)
        tensors = _plan_tensors(plan)

        fused = self._fused_activation(x)
        if fused == "swiglu":
            return _FusedSwiGLUExperts.apply(x, self.c_fc.weight, self.c_proj.weight, router_weights, *tensors,
                                             False, plan.row_dst)
        if fused == "swiglu_packed" and self._tensor_cores(x):
            # the interleaved epilogues exist on the tensor-core kernels only
            return _FusedSwiGLUExperts.apply(x, self.c_fc.weight, self.c_proj.weight, router_weights, *tensors,
                                             True, plan.row_dst)

        h = _UpProjectionExperts.apply(x, self.c_fc.weight, self.top_k, *tensors)
        h = self.act(h)
        return _DownProjectionExperts.apply(h, self.c_proj.weight, router_weights, *tensors)
