"""Auxiliary load-balancing loss on the `router_logits` that `xma.layers.MoE` returns.

The reference returns the logits unused (xma/layers/moe/__init__.py:180) and has no such loss; this is the usual
consumer a training loop adds (Switch Transformer, eq. 4-6, in the form used with top-k routing):

    loss = E * sum_e f_e * P_e,   P_e = mean_t softmax(logits)[t, e],   f_e = (slots routed to expert e) / tokens

with the same top-k rule as the layer (descending logit, lowest expert index first among equals). `f_e` is a count and
carries no gradient; the gradient flows through `P_e`. Two passes over `[tokens, E]` (csrc/aux_loss.cu) plus the routing
kernels the layer already uses for the counts."""

from __future__ import annotations

import torch

from .. import ops
from .._lib import require_cuda
from ..accelerator import KernelBackend
from .continuous_count import continuous_count

# rows of the per-CTA partial sums (CTAs of the forward kernel): 4 per SM of a B200, a constant so that nothing but
# tensor allocations and opaque custom ops sit in a traced graph
_PARTIAL_ROWS = 592


class _LoadBalancingLoss(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits: torch.Tensor, top_k: int) -> torch.Tensor:
        T, E = logits.shape
        weights = torch.empty(T, top_k, dtype=logits.dtype, device=logits.device)
        selected = torch.empty(T, top_k, dtype=torch.int32, device=logits.device)
        ops.route_topk_softmax_(logits, top_k, weights, selected)
        counts = continuous_count(selected.view(-1), E)
        frac = counts.view(torch.int32).to(torch.float32) / max(T, 1)
        partial = torch.empty(min(max(T, 1), _PARTIAL_ROWS), E, dtype=torch.float32, device=logits.device)
        ops.router_prob_sums_(logits, partial)
        mean_prob = partial.sum(0) / max(T, 1)
        ctx.save_for_backward(logits, frac)
        return (frac * mean_prob).sum() * E

    @staticmethod
    def backward(ctx, grad_out: torch.Tensor):
        logits, frac = ctx.saved_tensors
        T, E = logits.shape
        coef = (frac * (grad_out.to(torch.float32) * (E / max(T, 1)))).contiguous()
        d_logits = torch.empty(T, E, dtype=logits.dtype, device=logits.device)
        ops.load_balancing_loss_bwd_(logits, coef, d_logits)
        return d_logits, None


def load_balancing_loss(router_logits: torch.Tensor, num_experts_per_tok: int, *,
                        kernel_backend: KernelBackend | None = None) -> torch.Tensor:
    """`router_logits` [tokens, num_experts] (what `MoE.forward` returns second) -> fp32 scalar. Equals 1 x top_k for a
    perfectly uniform router (f_e = top_k / E, P_e = 1 / E) and grows as routing concentrates."""
    if kernel_backend not in (None, KernelBackend.cuda):
        raise ValueError(f"unexpected kernel_backend ({kernel_backend})")
    assert router_logits.dim() == 2, "router_logits should be 2D [tokens, num_experts]"
    assert 0 < num_experts_per_tok <= router_logits.size(1), "top-k must lie in [1, num_experts]"
    require_cuda(router_logits)
    if router_logits.size(1) > 1 and router_logits.stride(1) != 1:
        router_logits = router_logits.contiguous()
    return _LoadBalancingLoss.apply(router_logits, num_experts_per_tok)
