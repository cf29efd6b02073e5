"""Expert-parallel MoE over one process per GPU (torch.distributed, NCCL over NVLink).

The reference has no multi-GPU path (its MoE keeps all experts on one device,
xma/layers/moe/__init__.py:144-160); this is the sharding its data layout invites: rank r owns
experts [r*E/W, (r+1)*E/W), every rank routes its own tokens, and rows travel to the owner of their
expert and back:

    route (all E experts) -> count_sort by global expert id  (rows sorted by expert = sorted by owner)
    -> all_to_all of the per-expert counts                    (tiny, gives the split sizes)
    -> DISPATCH all_to_all of the sorted token rows           [R, H] -> [R_recv, H]
    -> local experts on the received rows (same kernels as the single-GPU layer, top_k = 1)
    -> COMBINE all_to_all back, then the weighted sum over the k slots on the home rank.

Routing weights are applied on the home rank, so only rows travel. Backward is the same exchange
with the roles of the splits swapped; expert weight gradients are rank-local. Received data always
lands in local HBM before a kernel reads it.

Overlap: with `overlap_chunks = C > 1` the rank's tokens are cut into C micro-batches that run the
whole path on alternating CUDA streams, so the all-to-alls of one micro-batch (NCCL's own stream)
run under the grouped GEMMs of the other; autograd replays the backward on the same streams, which
overlaps it the same way.
"""

from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn as nn

from . import ops
from .layers.moe import MoE, _FusedSwiGLUExperts, _plan_tensors, _TopKSoftmax, build_route_plan, SwiGLU


def split_sizes(counts: torch.Tensor, world: int) -> list[int]:
    """Rows per destination rank from per-expert counts [E] (E divisible by world)."""
    return counts.view(world, -1).sum(dim=1).tolist()


def exchange_counts(counts: torch.Tensor, group) -> torch.Tensor:
    """counts [E] of this rank -> [W, E_local]: row s = how many rows rank s sends to each local expert."""
    world = dist.get_world_size(group)
    recv = torch.empty_like(counts)
    dist.all_to_all_single(recv, counts.contiguous(), group=group)
    return recv.view(world, -1)


class _AllToAllRows(torch.autograd.Function):
    """Variable-size row exchange; the backward is the exchange with the splits swapped."""

    @staticmethod
    def forward(ctx, rows: torch.Tensor, send_splits: list[int], recv_splits: list[int], group):
        ctx.send_splits, ctx.recv_splits, ctx.group = send_splits, recv_splits, group
        out = rows.new_empty((sum(recv_splits), rows.size(1)))
        dist.all_to_all_single(out, rows.contiguous(), recv_splits, send_splits, group=group)
        return out

    @staticmethod
    def backward(ctx, grad: torch.Tensor):
        out = grad.new_empty((sum(ctx.send_splits), grad.size(1)))
        dist.all_to_all_single(out, grad.contiguous(), ctx.send_splits, ctx.recv_splits, group=ctx.group)
        return out, None, None, None


class _DispatchRows(torch.autograd.Function):
    """x [T, H] -> rows in expert-sorted order [R, H] (row p = token perm[p] // K)."""

    @staticmethod
    def forward(ctx, x: torch.Tensor, perm: torch.Tensor, inv_perm: torch.Tensor, top_k: int):
        out = x.new_empty((perm.numel(), x.size(1)))
        ops.gather_rows_(x, perm, None, top_k, None, out)
        ctx.save_for_backward(inv_perm)
        ctx.top_k, ctx.tokens = top_k, x.size(0)
        return out

    @staticmethod
    def backward(ctx, grad: torch.Tensor):
        (inv_perm,) = ctx.saved_tensors
        grad = grad.contiguous()
        dx = grad.new_empty((ctx.tokens, grad.size(1)))
        # sum of a token's K slots, read in place from the expert-sorted rows
        ops.combine_rows_(grad, None, ctx.top_k, dx, inv_perm)
        return dx, None, None, None


class _CombineRows(torch.autograd.Function):
    """expert-sorted rows [R, H], router_weights [T, K] -> y [T, H] = sum_k w[t,k] * row(t, k)."""

    @staticmethod
    def forward(ctx, rows: torch.Tensor, router_weights: torch.Tensor, perm: torch.Tensor, inv_perm: torch.Tensor):
        T, K = router_weights.shape
        rows = rows.contiguous()
        router_weights = router_weights.contiguous()
        y = rows.new_empty((T, rows.size(1)))
        ops.combine_rows_(rows, router_weights, K, y, inv_perm)
        ctx.save_for_backward(rows, router_weights, perm, inv_perm)
        return y

    @staticmethod
    def backward(ctx, dy: torch.Tensor):
        rows, router_weights, perm, inv_perm = ctx.saved_tensors
        T, K = router_weights.shape
        dy = dy.contiguous()
        d_rw = None
        if ctx.needs_input_grad[1]:
            d_rw = torch.empty_like(router_weights)
            ops.combine_bwd_(rows, dy, K, d_rw, inv_perm)
        d_rows = rows.new_empty(rows.shape)
        ops.gather_rows_(dy, perm, router_weights.view(-1), K, None, d_rows)
        return d_rows, d_rw, None, None


class ExpertParallelMoE(nn.Module):
    """Wraps a `MoE` that holds this rank's E/W experts (`c_fc`, `c_proj`) and a replicated router
    weight `[E, H]`. forward(x [.., H]) -> (y, router_logits [T, E]) for this rank's tokens."""

    def __init__(self, local_moe: MoE, gate_weight: torch.Tensor, world_group=None,
                 overlap_chunks: int | None = None) -> None:
        super().__init__()
        if not (isinstance(local_moe.act, SwiGLU) and local_moe.is_glu):
            raise ValueError("ExpertParallelMoE runs the fused SwiGLU expert block")
        self.local = local_moe
        self.group = world_group if world_group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.num_experts = local_moe.num_experts * self.world
        self.top_k = local_moe.top_k
        self.hidden_size = local_moe.hidden_size
        if tuple(gate_weight.shape) != (self.num_experts, self.hidden_size):
            raise ValueError("gate_weight must be [num_experts (global), hidden_size]")
        self.gate_weight = nn.Parameter(gate_weight.detach().clone())
        # exchange volume grows with (W-1)/W while the per-rank weight gradients (which every extra
        # micro-batch accumulates once more) shrink with 1/W: micro-batching pays from 4 ranks on
        self.overlap_chunks = overlap_chunks if overlap_chunks is not None else (2 if self.world >= 4 else 1)
        self._streams: list[torch.cuda.Stream] = []

    def forward(self, x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        original_shape = x.shape
        x = x.reshape(-1, self.hidden_size).contiguous()
        chunks = min(self.overlap_chunks, max(1, x.size(0)))
        if chunks <= 1:
            y, logits = self._forward_rows(x)
            return y.view(original_shape), logits
        if not self._streams:
            self._streams = [torch.cuda.Stream(device=x.device) for _ in range(2)]
        main = torch.cuda.current_stream(x.device)
        ys, logits = [], []
        for i, xc in enumerate(x.chunk(chunks, dim=0)):
            st = self._streams[i % 2]
            st.wait_stream(main)
            with torch.cuda.stream(st):
                y_i, l_i = self._forward_rows(xc)
            ys.append(y_i)
            logits.append(l_i)
        for st in self._streams:
            main.wait_stream(st)
        for t in ys + logits:
            t.record_stream(main)
        return torch.cat(ys, dim=0).view(original_shape), torch.cat(logits, dim=0)

    def _forward_rows(self, x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        E, K, W = self.num_experts, self.top_k, self.world
        e_local = E // W

        router_logits = torch.nn.functional.linear(x, self.gate_weight)
        router_weights, selected = _TopKSoftmax.apply(router_logits, K)

        with torch.no_grad():
            plan = build_route_plan(selected, E)
            perm = plan.sorted_scattered_idxs
            inv_perm = torch.empty_like(perm)
            inv_perm[perm.long()] = torch.arange(perm.numel(), dtype=torch.int32, device=perm.device)
            recv_counts = exchange_counts(plan.counts, self.group)  # [W, e_local]
            # one small device->host read per step: the split sizes NCCL needs on the host
            host = torch.cat([plan.counts.view(W, e_local).sum(1), recv_counts.sum(1)]).tolist()
            send_splits, recv_splits = host[:W], host[W:]
            # local expert id of every received row: source-major, expert-minor
            local_ids = torch.repeat_interleave(
                torch.arange(e_local, dtype=torch.int32, device=x.device).repeat(W), recv_counts.reshape(-1).long(),
                output_size=sum(recv_splits),
            )

        rows = _DispatchRows.apply(x, perm, inv_perm, K)
        recv = _AllToAllRows.apply(rows, send_splits, recv_splits, self.group)

        with torch.no_grad():
            local_plan = build_route_plan(local_ids.view(-1, 1), e_local)
        out = _FusedSwiGLUExperts.apply(recv, self.local.c_fc.weight, self.local.c_proj.weight, None,
                                        *_plan_tensors(local_plan))

        back = _AllToAllRows.apply(out, recv_splits, send_splits, self.group)
        y = _CombineRows.apply(back, router_weights, perm, inv_perm)
        return y, router_logits
