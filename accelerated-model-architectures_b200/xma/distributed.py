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

`transport="peer"` replaces the two row all-to-alls by stores into the other ranks' memory (the
ranks of one node map each other's exchange buffers once, CUDA IPC over NVLink):

    all_gather of the per-expert counts [W, E]  (tiny; one device->host read sizes the buffers)
    -> DISPATCH kernel: every routed token row is gathered and stored straight into its slot of the
       owner's padded, expert-major buffer, with a word naming its origin (home rank, token slot)
    -> barrier -> up projection + SwiGLU -> down projection whose epilogue stores every output row
       into its slot of the home rank's [T*K, H] buffer: GEMM and return exchange are one kernel
       (`fused_return=False`: a separate row kernel after a plain GEMM)
    -> barrier -> weighted sum over the k slots on the home rank.

Backward mirrors it (dY rows dispatched with the routing weight applied, dX rows returned the same
way). No kernel waits on another GPU: the phases are separated by a stream-ordered
barrier (a one-element NCCL all-reduce), so a rank that stops costs a collective timeout, never a
spinning kernel. What the backward needs of the exchanged rows stays in the exchange buffers (a second
pair of buffers serves the backward's exchange; `private_copies=True` copies instead), so a forward must
be followed by its backward before the next forward of the same layer.

Eager only: the exchange kernels write through raw addresses of other ranks' buffers (int64 tables), which
a tracing compiler cannot see as outputs of the ops; do not wrap this layer in `torch.compile`.
"""

from __future__ import annotations

import ctypes
import weakref

import numpy as np
import torch
import torch.distributed as dist
import torch.nn as nn

from . import ops
from ._lib import (EPI_DSWIGLU, EPI_PLAIN, EPI_SWIGLU, ROW_PAD, W_KN, W_NK, check, describe_device_status, lib,
                   status_word)
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


_PINNED: dict = {}


def _host_words(words: torch.Tensor):
    """int32 device tensor -> host numpy array (int64, same shape). A kernel stores the words into pinned
    host memory and the host waits on an event: unlike a device->host copy, the read does not queue in
    the copy engine behind bulk downloads of earlier steps."""
    if not words.is_cuda:
        return words.numpy().astype(np.int64)
    shape = tuple(words.shape)
    # the device status word rides along: this is the one host synchronisation of a step, so it is where a skipped
    # row, an expired wait or a bad tile table of the previous step's kernels surfaces as an exception
    status = status_word(words.device)
    words = torch.cat([words.reshape(-1), status])
    n = words.numel()
    pinned = _PINNED.get(words.device)
    if pinned is None or pinned.numel() < n:
        pinned = _PINNED[words.device] = torch.empty(max(n, 1024), dtype=torch.int32).pin_memory()
    stream = torch.cuda.current_stream(words.device)
    check(lib.xma_b200_ep_publish(words.data_ptr(), n, pinned.data_ptr(), stream.cuda_stream), "xma_b200_ep_publish")
    done = torch.cuda.Event()
    done.record(stream)
    done.synchronize()
    host = pinned[:n].numpy().astype(np.int64)
    if host[-1]:
        status.zero_()
        raise RuntimeError(describe_device_status(int(host[-1])) + " (results since the last check are undefined)")
    return host[:-1].reshape(shape)


# ---- peer-memory transport ---------------------------------------------------------------------------
class _DeviceBlock:
    """`cudaMalloc` memory of the current device, outside torch's caching allocator so that it can be
    exported to the other processes of the node; `tensor` is a uint8 view of it."""

    def __init__(self, nbytes: int, device: torch.device) -> None:
        out = ctypes.c_void_p()
        with torch.cuda.device(device):
            check(lib.xma_b200_exchange_alloc(nbytes, ctypes.byref(out)), "xma_b200_exchange_alloc")
        self.ptr, self.nbytes = int(out.value), int(nbytes)
        self.__cuda_array_interface__ = {
            "shape": (self.nbytes,), "typestr": "|u1", "data": (self.ptr, False), "version": 3, "strides": None,
        }
        self.tensor = torch.as_tensor(self, device=device)

    def export(self) -> bytes:
        handle = ctypes.create_string_buffer(lib.xma_b200_exchange_handle_bytes())
        check(lib.xma_b200_exchange_export(self.ptr, handle), "xma_b200_exchange_export")
        return handle.raw

    def free(self) -> None:
        if self.ptr:
            self.tensor = None
            check(lib.xma_b200_exchange_free(self.ptr), "xma_b200_exchange_free")
            self.ptr = 0


class PeerLink:
    """What the peer transport needs from the fabric, for the ranks of one node (one process per GPU):
    the count exchange, a barrier that orders the current stream after every rank's earlier work, and
    memory that every rank can store into."""

    def __init__(self, group) -> None:
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self._token: torch.Tensor | None = None

    def all_gather_counts(self, counts: torch.Tensor) -> torch.Tensor:
        out = torch.empty(self.world * counts.numel(), dtype=counts.dtype, device=counts.device)
        dist.all_gather_into_tensor(out, counts.contiguous(), group=self.group)
        return out.view(self.world, -1)

    def host_counts(self, count_matrix: torch.Tensor):
        """The count matrix as a host numpy array (int64)."""
        return _host_words(count_matrix)

    def barrier(self) -> None:
        if self._token is None:
            self._token = torch.zeros(1, dtype=torch.int32, device=torch.cuda.current_device())
        dist.all_reduce(self._token, group=self.group)

    def share(self, nbytes: int, device: torch.device):
        """Collective. -> (block of this rank, [address of every rank's block in this process], mapped addresses).
        A failure on any rank (allocation, export, mapping) raises on every rank, after the collectives."""
        block, handle, error = None, None, None
        try:
            block = _DeviceBlock(nbytes, device)
            handle = block.export()
        except Exception as exc:  # noqa: BLE001 - reported to every rank below
            error = repr(exc)
        handles: list = [None] * self.world
        dist.all_gather_object(handles, handle, group=self.group)
        addresses, mapped = [], []
        if error is None and all(h is not None for h in handles):
            try:
                with torch.cuda.device(device):
                    for r, peer_handle in enumerate(handles):
                        if r == self.rank:
                            addresses.append(block.ptr)
                            continue
                        out = ctypes.c_void_p()
                        check(lib.xma_b200_exchange_open(peer_handle, ctypes.byref(out)), "xma_b200_exchange_open")
                        addresses.append(int(out.value))
                        mapped.append(int(out.value))
            except Exception as exc:  # noqa: BLE001
                error = repr(exc)
        errors: list = [None] * self.world
        dist.all_gather_object(errors, error, group=self.group)  # also: everyone has mapped before anyone goes on
        if any(h is None for h in handles) or any(e is not None for e in errors):
            for address in mapped:
                lib.xma_b200_exchange_close(address)
            dist.barrier(group=self.group)
            if block is not None:
                block.free()
            raise RuntimeError(f"the ranks could not map each other's exchange buffers: {errors}")
        return block, addresses, mapped

    def release(self, block, mapped: list[int]) -> None:
        """Collective: nobody may still be storing into a block when its owner frees it."""
        torch.cuda.synchronize()
        dist.barrier(group=self.group)
        for address in mapped:
            check(lib.xma_b200_exchange_close(address), "xma_b200_exchange_close")
        dist.barrier(group=self.group)
        block.free()


def _round_up(value: int, multiple: int) -> int:
    return (value + multiple - 1) // multiple * multiple


class _Exchange:
    """Exchange buffers of one micro-batch slot, shared by every call of the layer:
    `recv_rows` [recv_cap, H] + `recv_meta` [recv_cap]: rows this rank's experts receive and where each
    came from; `home_rows` [home_cap, H]: expert outputs returned to this rank, one row per token slot.
    `*_table`: int64 [W] device tensors with every rank's address of the same buffer."""

    def __init__(self, link, device: torch.device, dtype: torch.dtype, hidden: int, fused_return: bool,
                 private_copies: bool = False) -> None:
        self.link, self.device, self.dtype, self.hidden = link, device, dtype, hidden
        self.fused_return = fused_return
        self.private_copies = private_copies
        self.recv_cap = self.home_cap = 0
        self._held: list = []
        self.recv_rows = self.recv_meta = self.home_rows = None
        self.recv_table = self.meta_table = self.home_table = None
        # Without private copies the forward's received rows and returned rows stay in the exchange buffers
        # until the backward has read them, and the backward exchanges through a second pair of buffers.
        self.recv_rows_bwd = self.home_rows_bwd = None
        self.recv_table_bwd = self.home_table_bwd = None
        self._in_use = None  # weak reference to the forward whose tensors live in the buffers
        self._side = None

    def side_stream(self, device: torch.device) -> torch.cuda.Stream:
        """The stream the dispatches of the pipelined exchange are queued on."""
        if self._side is None:
            self._side = torch.cuda.Stream(device=device)
        return self._side

    def claim(self, owner) -> None:
        """The forward `owner` is about to fill the forward buffers. An earlier forward whose backward has not
        run yet still needs them: peers would overwrite its rows, and no local copy could be ordered before
        their stores without one more barrier, so that use is refused."""
        if self.private_copies:
            return
        previous = self._in_use() if self._in_use is not None else None
        if previous is not None and not previous.done:
            raise RuntimeError(
                "ExpertParallelMoE(transport='peer'): a second forward started before the backward of the previous "
                "one; its saved rows live in the exchange buffers. Construct the layer with private_copies=True "
                "to run several forwards before their backwards (one extra copy of the received and returned rows)")
        self._in_use = weakref.ref(owner) if owner is not None else None

    def _shared(self, nbytes: int):
        block, addresses, mapped = self.link.share(nbytes, self.device)
        self._held.append((block, mapped))
        return block.tensor, torch.tensor(addresses, dtype=torch.int64, device=self.device)

    def ensure(self, need_recv: int, need_home: int) -> None:
        """Collective whenever it reallocates; every rank calls it with the same arguments."""
        if need_recv <= self.recv_cap and need_home <= self.home_cap:
            return
        if max(need_recv, need_home) > (1 << 24):
            raise ValueError("the peer transport addresses at most 2^24 rows per rank")
        self.close()
        item = torch.empty((), dtype=self.dtype).element_size()
        self.recv_cap = max(self.recv_cap, _round_up(need_recv + need_recv // 4, ROW_PAD), ROW_PAD)
        self.home_cap = max(self.home_cap, _round_up(need_home + need_home // 4, ROW_PAD), ROW_PAD)
        raw, self.recv_table = self._shared(self.recv_cap * self.hidden * item)
        self.recv_rows = raw.view(self.dtype).view(self.recv_cap, self.hidden)
        raw, self.meta_table = self._shared(self.recv_cap * 4)
        self.recv_meta = raw.view(torch.int32)
        raw, self.home_table = self._shared(self.home_cap * self.hidden * item)
        self.home_rows = raw.view(self.dtype).view(self.home_cap, self.hidden)
        if self.private_copies:
            self.recv_rows_bwd, self.recv_table_bwd = self.recv_rows, self.recv_table
            self.home_rows_bwd, self.home_table_bwd = self.home_rows, self.home_table
        else:
            raw, self.recv_table_bwd = self._shared(self.recv_cap * self.hidden * item)
            self.recv_rows_bwd = raw.view(self.dtype).view(self.recv_cap, self.hidden)
            raw, self.home_table_bwd = self._shared(self.home_cap * self.hidden * item)
            self.home_rows_bwd = raw.view(self.dtype).view(self.home_cap, self.hidden)

    def close(self) -> None:
        """Collective."""
        self.recv_rows = self.recv_meta = self.home_rows = self.recv_rows_bwd = self.home_rows_bwd = None
        for block, mapped in self._held:
            self.link.release(block, mapped)
        self._held = []


class _PeerRoute:
    """Device tables of one routing decision under the peer transport (all from `ep_plan`), and the host's view
    of how this rank's experts are cut into the parts of the pipelined exchange."""

    def __init__(self, count_matrix: torch.Tensor, rank: int, rows: int, exchange: _Exchange,
                 local_padded=None, parts: int = 1) -> None:
        world, num_experts = count_matrix.shape
        e_local = num_experts // world
        dev = count_matrix.device
        self.world, self.rank, self.rows, self.e_local = world, rank, rows, e_local
        sizes = (num_experts, e_local, e_local + 1, e_local + 1, rows // ROW_PAD + e_local)
        (self.send_delta, self.counts, self.pad_offsets, self.tile_prefix,
         self.tile_expert) = torch.empty(sum(sizes), dtype=torch.int32, device=dev).split(sizes)
        ops.ep_plan_(count_matrix, rank, self.send_delta, self.counts, self.pad_offsets, self.tile_prefix,
                     self.tile_expert, exchange.recv_meta)
        # parts: (first local expert, one past the last, first padded row, one past the last) - contiguous groups
        # of this rank's experts; `local_padded` = padded rows of each local expert, known to the host
        parts = max(1, min(int(parts), e_local))
        if local_padded is None or parts == 1:
            self.parts = [(0, e_local, 0, rows)]
        else:
            ends = np.concatenate([[0], np.cumsum(np.asarray(local_padded, dtype=np.int64))])
            cuts = [round(i * e_local / parts) for i in range(parts + 1)]
            self.parts = [(cuts[i], cuts[i + 1], int(ends[cuts[i]]), int(ends[cuts[i + 1]])) for i in range(parts)]


class _KeptRows:
    """Tensors of one forward that the backward reads: the rows this rank's experts received (`xs`) and the
    expert outputs returned to this rank (`ys`): private copies, or views of the exchange buffers."""

    __slots__ = ("xs", "ys", "done", "__weakref__")

    def __init__(self) -> None:
        self.xs = self.ys = None
        self.done = False


class _PeerSwiGLUExperts(torch.autograd.Function):
    """The fused SwiGLU expert block with the experts sharded over the ranks: dispatch and combine are
    stores into the other ranks' exchange buffers (see the module docstring).

    The exchange is pipelined by expert: this rank's experts are cut into `route.parts` contiguous groups, every
    rank dispatches the rows of group 0, then of group 1, ... on a side stream (each followed by a barrier over
    the ranks), and the main stream runs the grouped GEMMs of a group as soon as its rows have landed - the
    dispatch of group i + 1 travels under the GEMMs of group i. The GEMMs are whole experts either way, so
    nothing is computed twice (cutting the tokens instead would add every weight gradient up once per cut)."""

    @staticmethod
    def _dispatch_parts(src, coeff, K, sorted_expert_idxs, sorted_scattered_idxs, route, exchange, recv_table,
                        meta_table):
        """Queues every part's dispatch + barrier on the exchange's side stream; -> one event per part."""
        main = torch.cuda.current_stream(src.device)
        side = exchange.side_stream(src.device)
        side.wait_stream(main)
        events = []
        with torch.cuda.stream(side):
            for lo, hi, _, _ in route.parts:
                ops.ep_dispatch_(src, sorted_expert_idxs, sorted_scattered_idxs, coeff, K, route.send_delta,
                                 route.world, route.rank, recv_table, meta_table, exchange.recv_cap, lo, hi)
                exchange.link.barrier()
                ev = torch.cuda.Event()
                ev.record(side)
                events.append(ev)
        for t in (src, coeff):
            if t is not None:
                t.record_stream(side)
        return events

    @staticmethod
    def forward(ctx, x, router_weights, w1, w2, sorted_expert_idxs, sorted_scattered_idxs, route, exchange):
        T, K = router_weights.shape
        e_local, two_i, H = w1.shape
        I = two_i // 2
        R = T * K
        link = exchange.link
        opts = dict(dtype=x.dtype, device=x.device)
        impl = ops.GEMM_IMPL
        rows = route.rows                              # padded rows of this rank's experts in use
        alloc = route.tile_expert.numel() * ROW_PAD    # grouped buffers span the whole tile table
        main = torch.cuda.current_stream(x.device)

        kept = _KeptRows() if any(ctx.needs_input_grad) else None
        exchange.claim(kept)
        arrived = _PeerSwiGLUExperts._dispatch_parts(x, None, K, sorted_expert_idxs, sorted_scattered_idxs, route,
                                                     exchange, exchange.recv_table, exchange.meta_table)

        meta = torch.full((alloc,), -1, dtype=torch.int32, device=x.device)
        xs = torch.empty(alloc, H, **opts) if exchange.private_copies else exchange.recv_rows[:alloc]
        gu = torch.empty(alloc, two_i, **opts)
        act = torch.empty(alloc, I, **opts)
        out = None if exchange.fused_return else torch.empty(alloc, H, **opts)
        for (lo, hi, r0, r1), ev in zip(route.parts, arrived):
            main.wait_event(ev)
            meta[r0:r1].copy_(exchange.recv_meta[r0:r1])
            if exchange.private_copies:
                ops.ep_copy_rows_(exchange.recv_rows[r0:r1], meta[r0:r1], xs[r0:r1])
            else:
                ops.ep_copy_rows_(xs[r0:r1], meta[r0:r1], xs[r0:r1])  # in place: zero the pad rows
            tiles = route.tile_prefix[lo:hi + 1]
            ops.grouped_gemm_rows_(xs, w1[lo:hi], W_NK, act, gu, None, route.tile_expert, tiles, H, two_i,
                                   EPI_SWIGLU, impl, tag="gemm_up_swiglu")
            if exchange.fused_return:
                ops.grouped_gemm_rows_(act, w2[lo:hi], W_NK, exchange.home_rows, None, meta, route.tile_expert,
                                       tiles, I, H, EPI_PLAIN, impl, exchange.home_table, exchange.home_cap,
                                       tag="gemm_down")
            else:
                ops.grouped_gemm_rows_(act, w2[lo:hi], W_NK, out, None, None, route.tile_expert, tiles, I, H,
                                       EPI_PLAIN, impl, tag="gemm_down")
        if not exchange.fused_return:
            ops.ep_return_(out[:rows], meta, route.world, exchange.home_table, exchange.home_cap)
        link.barrier()

        ys = exchange.home_rows[:R].clone() if exchange.private_copies else exchange.home_rows[:R]
        y = torch.empty(T, H, **opts)
        router_weights = router_weights.contiguous()
        if T > 0:
            ops.combine_rows_(ys, router_weights, K, y)
        ctx.save_for_backward(gu, act, meta, w1, w2, router_weights, sorted_expert_idxs, sorted_scattered_idxs)
        if kept is not None:
            kept.xs, kept.ys = xs, ys
        ctx.route, ctx.exchange, ctx.kept = route, exchange, kept
        return y

    @staticmethod
    def backward(ctx, grad_out):
        gu, act, meta, w1, w2, router_weights, sorted_expert_idxs, sorted_scattered_idxs = ctx.saved_tensors
        route, exchange, kept = ctx.route, ctx.exchange, ctx.kept
        xs, ys = kept.xs, kept.ys
        link = exchange.link
        T, K = router_weights.shape
        e_local, two_i, H = w1.shape
        I = two_i // 2
        R = T * K
        rows = route.rows
        alloc = xs.size(0)
        opts = dict(dtype=xs.dtype, device=xs.device)
        impl = ops.GEMM_IMPL
        grad_out = grad_out.contiguous()
        main = torch.cuda.current_stream(xs.device)

        # dY rows, scaled by their routing weight, to the owners (same slots as the forward rows), part by part
        arrived = _PeerSwiGLUExperts._dispatch_parts(grad_out, router_weights.view(-1), K, sorted_expert_idxs,
                                                     sorted_scattered_idxs, route, exchange,
                                                     exchange.recv_table_bwd, None)
        d_rw = None
        if ctx.needs_input_grad[1]:
            d_rw = torch.empty_like(router_weights)
            if T > 0:
                ops.combine_bwd_(ys, grad_out, K, d_rw)

        dys = exchange.recv_rows_bwd[:alloc]
        d_w1, d_w2 = torch.empty_like(w1), torch.empty_like(w2)
        dgu = torch.empty(alloc, two_i, **opts)
        dxs = None if exchange.fused_return else torch.empty(alloc, H, **opts)
        for (lo, hi, r0, r1), ev in zip(route.parts, arrived):
            main.wait_event(ev)
            ops.ep_copy_rows_(dys[r0:r1], meta[r0:r1], dys[r0:r1])  # in place: zero the pad rows
            tiles, counts, pads = route.tile_prefix[lo:hi + 1], route.counts[lo:hi], route.pad_offsets[lo:hi + 1]
            ops.grouped_gemm_dw_(dys, act, counts, pads, d_w2[lo:hi], impl, tag="gemm_dw2")
            ops.grouped_gemm_rows_(dys, w2[lo:hi], W_KN, dgu, gu, None, route.tile_expert, tiles, H, I, EPI_DSWIGLU,
                                   impl, tag="gemm_dact_dswiglu")
            ops.grouped_gemm_dw_(dgu, xs, counts, pads, d_w1[lo:hi], impl, tag="gemm_dw1")
            # dX rows straight back to the token's home rank
            if exchange.fused_return:
                ops.grouped_gemm_rows_(dgu, w1[lo:hi], W_KN, exchange.home_rows_bwd, None, meta, route.tile_expert,
                                       tiles, two_i, H, EPI_PLAIN, impl, exchange.home_table_bwd, exchange.home_cap,
                                       tag="gemm_dx")
            else:
                ops.grouped_gemm_rows_(dgu, w1[lo:hi], W_KN, dxs, None, None, route.tile_expert, tiles, two_i, H,
                                       EPI_PLAIN, impl, tag="gemm_dx")
        if not exchange.fused_return:
            ops.ep_return_(dxs[:rows], meta, route.world, exchange.home_table_bwd, exchange.home_cap)
        # every read of the forward's rows (xs for dW1, ys for d_router_weights) is queued in front of this
        # barrier, so the buffers are free for the next forward once it has passed
        kept.done = True
        link.barrier()

        d_x = torch.empty(T, H, **opts)
        if T > 0:
            ops.combine_rows_(exchange.home_rows_bwd[:R], None, K, d_x)
        return d_x, d_rw, d_w1, d_w2, None, None, None, None


class ExpertParallelMoE(nn.Module):
    """Wraps a `MoE` that holds this rank's E/W experts (`c_fc`, `c_proj`) and a replicated router
    weight `[E, H]`. forward(x [.., H]) -> (y, router_logits [T, E]) for this rank's tokens."""

    def __init__(self, local_moe: MoE, gate_weight: torch.Tensor, world_group=None,
                 overlap_chunks: int | None = None, transport: str = "nccl", link=None,
                 fused_return: bool = True, private_copies: bool = False, pipeline_parts: int | None = None) -> None:
        """`transport`: "nccl" (all-to-all collectives; any process group) or "peer" (stores into the
        other ranks' memory; the ranks must be GPUs of one node with peer access). `link` replaces the
        `PeerLink` built from the process group (the tests run several ranks on one GPU with it).
        `fused_return` (peer transport): the down-projection and dX GEMMs store their rows into the home
        ranks' memory from their own epilogues (GEMM and exchange are one kernel; the tile is staged in
        shared memory so that each row leaves in 128-byte pieces); False runs a separate row kernel.
        `private_copies` (peer transport): False keeps what the backward needs of the exchanged rows in the
        exchange buffers themselves (the backward exchanges through a second pair of buffers), which saves two
        passes over `[rows, hidden]` per step but allows one forward per backward at a time; True copies them.
        `pipeline_parts` (peer transport): this rank's experts are cut into that many groups and the rows of one
        group are dispatched while the GEMMs of the previous one run (default 1: the exchange in one piece)."""
        super().__init__()
        if not (getattr(local_moe.act, "xma_fused_activation", None) == "swiglu" and local_moe.is_glu):
            raise ValueError("ExpertParallelMoE runs the fused SwiGLU expert block")
        if transport not in ("nccl", "peer"):
            raise ValueError("transport must be 'nccl' or 'peer'")
        self.local = local_moe
        self.transport = transport
        self.fused_return = fused_return
        self.private_copies = private_copies
        self.pipeline_parts = pipeline_parts
        if link is not None:
            self.link, self.group = link, None
            self.world, self.rank = link.world, link.rank
        else:
            self.group = world_group if world_group is not None else dist.group.WORLD
            self.world = dist.get_world_size(self.group)
            self.rank = dist.get_rank(self.group)
            self.link = PeerLink(self.group) if transport == "peer" else None
        self._exchanges: dict = {}
        self.num_experts = local_moe.num_experts * self.world
        self.top_k = local_moe.top_k
        self.hidden_size = local_moe.hidden_size
        if tuple(gate_weight.shape) != (self.num_experts, self.hidden_size):
            raise ValueError("gate_weight must be [num_experts (global), hidden_size]")
        self.gate_weight = nn.Parameter(gate_weight.detach().clone())
        # exchange volume grows with (W-1)/W while the per-rank weight gradients (which every extra
        # micro-batch accumulates once more) shrink with 1/W: micro-batching pays from 4 ranks on
        # (the peer transport hides the way back inside the GEMMs, so it starts from one micro-batch)
        if overlap_chunks is None:
            overlap_chunks = 2 if (self.world >= 4 and transport == "nccl") else 1
        self.overlap_chunks = overlap_chunks
        self._streams: list[torch.cuda.Stream] = []

    def forward(self, x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        original_shape = x.shape
        x = x.reshape(-1, self.hidden_size).contiguous()
        chunks = min(self.overlap_chunks, max(1, x.size(0)))
        if chunks <= 1:
            y, logits = self._forward_rows(x, 0)
            return y.view(original_shape), logits
        if not self._streams:
            self._streams = [torch.cuda.Stream(device=x.device) for _ in range(2)]
        main = torch.cuda.current_stream(x.device)
        ys, logits = [], []
        for i, xc in enumerate(x.chunk(chunks, dim=0)):
            st = self._streams[i % 2]
            st.wait_stream(main)
            with torch.cuda.stream(st):
                y_i, l_i = self._forward_rows(xc, i % 2)
            ys.append(y_i)
            logits.append(l_i)
        for st in self._streams:
            main.wait_stream(st)
        for t in ys + logits:
            t.record_stream(main)
        return torch.cat(ys, dim=0).view(original_shape), torch.cat(logits, dim=0)

    def _exchange(self, slot: int, x: torch.Tensor) -> _Exchange:
        key = (slot, x.device, x.dtype)
        if key not in self._exchanges:
            self._exchanges[key] = _Exchange(self.link, x.device, x.dtype, self.hidden_size, self.fused_return,
                                             self.private_copies)
        return self._exchanges[key]

    def close(self) -> None:
        """Collective: unmaps and frees the exchange buffers of the peer transport."""
        for exchange in self._exchanges.values():
            exchange.close()
        self._exchanges = {}

    def _forward_rows_peer(self, x: torch.Tensor, slot: int) -> tuple[torch.Tensor, torch.Tensor]:
        E, K, W = self.num_experts, self.top_k, self.world
        e_local = E // W
        router_logits = torch.nn.functional.linear(x, self.gate_weight)
        router_weights, selected = _TopKSoftmax.apply(router_logits, K)
        with torch.no_grad():
            plan = build_route_plan(selected, E)
            count_matrix = self.link.all_gather_counts(plan.counts)  # [W, E] int32
            # one small device->host read per step: every rank sizes every rank's buffers from it,
            # so all of them take the same (collective) decision to grow the exchange buffers
            host = self.link.host_counts(count_matrix)
            padded = ((host.sum(0) + ROW_PAD - 1) // ROW_PAD * ROW_PAD).reshape(W, e_local).sum(1)
            exchange = self._exchange(slot, x)
            # (grouped buffers are allocated for rows // 128 + e_local tiles, the received rows included)
            exchange.ensure(int(padded.max()) + e_local * ROW_PAD, int(host.sum(1).max()))
            local_padded = ((host.sum(0) + ROW_PAD - 1) // ROW_PAD * ROW_PAD)[self.rank * e_local:
                                                                                (self.rank + 1) * e_local]
            parts = self.pipeline_parts if self.pipeline_parts is not None else 1
            if not self.local._tensor_cores(x):
                parts = 1  # the CUDA-core GEMMs take whole tile tables only
            route = _PeerRoute(count_matrix, self.rank, int(padded[self.rank]), exchange, local_padded, parts)
        y = _PeerSwiGLUExperts.apply(x, router_weights, self.local.c_fc.weight, self.local.c_proj.weight,
                                     plan.sorted_expert_idxs, plan.sorted_scattered_idxs, route, exchange)
        return y, router_logits

    def _forward_rows(self, x: torch.Tensor, slot: int = 0) -> tuple[torch.Tensor, torch.Tensor]:
        if self.transport == "peer":
            return self._forward_rows_peer(x, slot)
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
            host = _host_words(torch.cat([plan.counts.view(W, e_local).sum(1), recv_counts.sum(1)]).to(torch.int32))
            send_splits, recv_splits = host[:W].tolist(), host[W:].tolist()
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
