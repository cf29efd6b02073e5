"""`torch.library` custom ops over the C ABI (namespace `xma_b200::`).

Same convention as the reference's `xma_op` (xma/custom_op.py:72-108): the caller allocates every
output with torch, the op mutates it and returns None, so no fake implementation is needed and the
ops trace under `torch.compile(fullgraph=True)`. Each op forwards raw device pointers, sizes and
the current CUDA stream to one `extern "C"` function of libxma_b200.so.
"""

from __future__ import annotations

import os
from typing import Optional

import torch
from torch import Tensor

from . import _lib
from ._lib import check, current_stream, dtype_code, lib, ptr, require_cuda, status_word

_NS = "xma_b200"


def _row_stride(t: Tensor) -> int:
    if t.dim() != 2 or (t.size(1) > 1 and t.stride(1) != 1):
        raise ValueError("expected a 2-D tensor whose last dimension is contiguous")
    return t.stride(0) if t.size(0) > 1 else max(t.stride(0), t.size(1))


@torch.library.custom_op(f"{_NS}::continuous_count", mutates_args={"counts"}, device_types="cuda")
def _continuous_count_op(ids: Tensor, counts: Tensor) -> None:
    require_cuda(ids, counts)
    check(
        lib.xma_b200_continuous_count(
            ptr(ids), dtype_code(ids.dtype), ids.numel(), counts.numel(), ptr(counts), ptr(status_word(ids.device)),
            current_stream(ids.device)
        ),
        "xma_b200_continuous_count",
    )


@torch.library.custom_op(f"{_NS}::route_topk_softmax", mutates_args={"weights", "selected"}, device_types="cuda")
def _route_topk_softmax_op(logits: Tensor, top_k: int, weights: Tensor, selected: Tensor) -> None:
    require_cuda(logits, weights, selected)
    sel32 = ptr(selected) if selected.dtype == torch.int32 else None
    sel64 = ptr(selected) if selected.dtype == torch.int64 else None
    check(
        lib.xma_b200_route_topk_softmax(
            ptr(logits), dtype_code(logits.dtype), _row_stride(logits), logits.size(0), logits.size(1), top_k,
            ptr(weights), sel32, sel64, current_stream(logits.device)
        ),
        "xma_b200_route_topk_softmax",
    )


@torch.library.custom_op(f"{_NS}::route_topk_softmax_bwd", mutates_args={"d_logits"}, device_types="cuda")
def _route_topk_softmax_bwd_op(logits: Tensor, selected: Tensor, d_weights: Tensor, d_logits: Tensor) -> None:
    require_cuda(logits, selected, d_weights, d_logits)
    check(
        lib.xma_b200_route_topk_softmax_bwd(
            ptr(logits), dtype_code(logits.dtype), _row_stride(logits), ptr(selected), ptr(d_weights),
            logits.size(0), logits.size(1), selected.size(1), ptr(d_logits), current_stream(logits.device)
        ),
        "xma_b200_route_topk_softmax_bwd",
    )


@torch.library.custom_op(
    f"{_NS}::count_sort",
    mutates_args={"counts", "offsets_incl", "pad_offsets", "tile_prefix", "tile_expert", "sorted_expert_idxs",
                  "sorted_scattered_idxs", "row_src"},
    device_types="cuda",
)
def _count_sort_op(
    ids: Tensor,
    num_experts: int,
    counts: Tensor,
    offsets_incl: Tensor,
    pad_offsets: Tensor,
    tile_prefix: Tensor,
    tile_expert: Tensor,
    sorted_expert_idxs: Tensor,
    sorted_scattered_idxs: Tensor,
    row_src: Tensor,
    row_dst: Optional[Tensor] = None,
) -> None:
    require_cuda(ids)
    n = ids.numel()
    scratch_bytes = lib.xma_b200_count_sort_scratch_bytes(n, num_experts)
    if scratch_bytes < 0:
        check(int(scratch_bytes), "xma_b200_count_sort_scratch_bytes")
    scratch = torch.empty(scratch_bytes, dtype=torch.uint8, device=ids.device)
    check(
        lib.xma_b200_count_sort(
            ptr(ids), dtype_code(ids.dtype), n, num_experts, ptr(counts), ptr(offsets_incl), ptr(pad_offsets),
            ptr(tile_prefix), ptr(tile_expert), tile_expert.numel(), ptr(sorted_expert_idxs),
            ptr(sorted_scattered_idxs), ptr(row_src), row_src.numel(), ptr(row_dst), ptr(scratch), scratch_bytes,
            ptr(status_word(ids.device)), current_stream(ids.device)
        ),
        "xma_b200_count_sort",
    )


@torch.library.custom_op(f"{_NS}::gather_rows", mutates_args={"out"}, device_types="cuda")
def _gather_rows_op(
    src: Tensor, row_src: Tensor, coeff: Optional[Tensor], fan_out: int, rows_in_use: Optional[Tensor], out: Tensor
) -> None:
    require_cuda(src, row_src, out)
    check(
        lib.xma_b200_gather_rows(
            ptr(src), dtype_code(src.dtype), _row_stride(src), ptr(row_src), ptr(coeff), fan_out, out.size(0),
            ptr(rows_in_use), src.size(1), ptr(out), _row_stride(out), current_stream(src.device)
        ),
        "xma_b200_gather_rows",
    )


@torch.library.custom_op(f"{_NS}::spread_rows", mutates_args={"out", "d_weights"}, device_types="cuda")
def _spread_rows_op(src: Tensor, row_dst: Tensor, coeff: Optional[Tensor], ys: Optional[Tensor],
                    d_weights: Optional[Tensor], top_k: int, counts: Tensor, pad_offsets: Tensor, out: Tensor) -> None:
    require_cuda(src, row_dst, out)
    check(
        lib.xma_b200_spread_rows(
            ptr(src), dtype_code(src.dtype), _row_stride(src), ptr(row_dst), ptr(coeff), ptr(ys),
            0 if ys is None else _row_stride(ys), ptr(d_weights), top_k, src.size(0), src.size(1), ptr(out),
            _row_stride(out), ptr(counts), ptr(pad_offsets), counts.numel(), current_stream(src.device)
        ),
        "xma_b200_spread_rows",
    )


@torch.library.custom_op(f"{_NS}::combine_rows", mutates_args={"y"}, device_types="cuda")
def _combine_rows_op(ys: Tensor, weights: Optional[Tensor], top_k: int, y: Tensor,
                     row_index: Optional[Tensor] = None) -> None:
    require_cuda(ys, y)
    check(
        lib.xma_b200_combine_rows(
            ptr(ys), dtype_code(ys.dtype), _row_stride(ys), ptr(weights), ptr(row_index), top_k, y.size(0),
            y.size(1), ptr(y), _row_stride(y), current_stream(ys.device)
        ),
        "xma_b200_combine_rows",
    )


@torch.library.custom_op(f"{_NS}::combine_bwd", mutates_args={"d_weights"}, device_types="cuda")
def _combine_bwd_op(ys: Tensor, dy: Tensor, top_k: int, d_weights: Tensor,
                    row_index: Optional[Tensor] = None) -> None:
    require_cuda(ys, dy, d_weights)
    check(
        lib.xma_b200_combine_bwd(
            ptr(ys), dtype_code(ys.dtype), _row_stride(ys), ptr(dy), _row_stride(dy), ptr(row_index), top_k,
            dy.size(0), dy.size(1), ptr(d_weights), current_stream(ys.device)
        ),
        "xma_b200_combine_bwd",
    )


@torch.library.custom_op(f"{_NS}::grouped_gemm_rows", mutates_args={"out", "aux"}, device_types="cuda")
def _grouped_gemm_rows_op(
    a: Tensor,
    w: Tensor,
    w_layout: int,
    out: Tensor,
    aux: Optional[Tensor],
    row_map: Optional[Tensor],
    tile_expert: Tensor,
    tile_prefix: Tensor,
    kd: int,
    n: int,
    epilogue: int,
    impl: int,
    out_peers: Optional[Tensor] = None,
    peer_rows_cap: int = 0,
) -> None:
    """`out_peers` (int64 [world], device): base address of every rank's output buffer of `peer_rows_cap`
    rows; rows then go to the rank named by `row_map` (expert parallelism) and `out` is this rank's own
    buffer. A word of `row_map` that names a rank or a row outside them is skipped and sets status bit 1."""
    require_cuda(a, w, out)
    if out_peers is not None and peer_rows_cap <= 0:
        raise ValueError("out_peers needs peer_rows_cap, the number of rows of every rank's buffer")
    if not w.is_contiguous():
        raise ValueError("expert weights must be contiguous [E, out_features, in_features]")
    check(
        lib.xma_b200_grouped_gemm_rows_peer(
            ptr(a), _row_stride(a), ptr(w), w_layout, ptr(out), _row_stride(out), ptr(aux),
            0 if aux is None else _row_stride(aux), ptr(row_map), ptr(out_peers),
            0 if out_peers is None else out_peers.numel(), peer_rows_cap, ptr(tile_expert), ptr(tile_prefix),
            w.size(0), tile_expert.numel(), kd, n, epilogue, dtype_code(a.dtype), impl, ptr(status_word(a.device)),
            current_stream(a.device)
        ),
        "xma_b200_grouped_gemm_rows",
    )


@torch.library.custom_op(f"{_NS}::grouped_gemm_dw", mutates_args={"dw"}, device_types="cuda")
def _grouped_gemm_dw_op(x: Tensor, y: Tensor, counts: Tensor, pad_offsets: Tensor, dw: Tensor, impl: int) -> None:
    require_cuda(x, y, dw)
    check(
        lib.xma_b200_grouped_gemm_dw(
            ptr(x), _row_stride(x), ptr(y), _row_stride(y), ptr(counts), ptr(pad_offsets), x.size(0), dw.size(0),
            dw.size(1), dw.size(2), ptr(dw), dtype_code(x.dtype), impl, ptr(status_word(x.device)),
            current_stream(x.device)
        ),
        "xma_b200_grouped_gemm_dw",
    )


@torch.library.custom_op(
    f"{_NS}::ep_plan",
    mutates_args={"send_delta", "counts", "pad_offsets", "tile_prefix", "tile_expert", "meta"},
    device_types="cuda",
)
def _ep_plan_op(count_matrix: Tensor, rank: int, send_delta: Tensor, counts: Tensor, pad_offsets: Tensor,
                tile_prefix: Tensor, tile_expert: Tensor, meta: Tensor) -> None:
    require_cuda(count_matrix, send_delta, meta)
    if count_matrix.dtype != torch.int32 or not count_matrix.is_contiguous():
        raise ValueError("count_matrix must be a contiguous int32 [world, num_experts] tensor")
    check(
        lib.xma_b200_ep_plan(
            ptr(count_matrix), count_matrix.size(0), count_matrix.size(1), rank, ptr(send_delta), ptr(counts),
            ptr(pad_offsets), ptr(tile_prefix), ptr(tile_expert), tile_expert.numel(), ptr(meta), meta.numel(),
            ptr(status_word(meta.device)), current_stream(meta.device)
        ),
        "xma_b200_ep_plan",
    )


@torch.library.custom_op(f"{_NS}::ep_dispatch", mutates_args=(), device_types="cuda")
def _ep_dispatch_op(src: Tensor, sorted_expert_idxs: Tensor, sorted_scattered_idxs: Tensor, coeff: Optional[Tensor],
                    fan_out: int, send_delta: Tensor, world: int, rank: int, peer_rows: Tensor,
                    peer_meta: Optional[Tensor], peer_rows_cap: int, local_lo: int = 0, local_hi: int = -1) -> None:
    """Writes into the exchange buffers whose addresses `peer_rows` / `peer_meta` (int64 [world]) hold; only the rows
    for the owners' local experts [local_lo, local_hi) (all of them by default)."""
    require_cuda(src, sorted_expert_idxs, sorted_scattered_idxs, send_delta, peer_rows)
    if local_hi < 0:
        local_hi = send_delta.numel() // world
    check(
        lib.xma_b200_ep_dispatch_part(
            ptr(src), dtype_code(src.dtype), _row_stride(src), ptr(sorted_expert_idxs), ptr(sorted_scattered_idxs),
            ptr(coeff), fan_out, ptr(send_delta), send_delta.numel(), world, rank, local_lo, local_hi,
            sorted_expert_idxs.numel(), src.size(1), ptr(peer_rows), ptr(peer_meta), peer_rows_cap,
            ptr(status_word(src.device)), current_stream(src.device)
        ),
        "xma_b200_ep_dispatch",
    )


@torch.library.custom_op(f"{_NS}::ep_copy_rows", mutates_args={"out"}, device_types="cuda")
def _ep_copy_rows_op(rows: Tensor, meta: Tensor, out: Tensor) -> None:
    """out[r] = rows[r] where meta[r] >= 0, zeros elsewhere, for the out.size(0) first rows
    (`out` may be `rows` itself: only the pad rows are then written)."""
    require_cuda(rows, meta, out)
    if not (rows.is_contiguous() and out.is_contiguous()):
        raise ValueError("exchange rows must be dense")
    check(
        lib.xma_b200_ep_copy_rows(ptr(rows), dtype_code(rows.dtype), ptr(meta), out.size(0), out.size(1), ptr(out),
                                  current_stream(rows.device)),
        "xma_b200_ep_copy_rows",
    )


@torch.library.custom_op(f"{_NS}::ep_return", mutates_args=(), device_types="cuda")
def _ep_return_op(rows: Tensor, meta: Tensor, world: int, peer_rows: Tensor, peer_rows_cap: int) -> None:
    """Stores every row whose origin word is >= 0 into the exchange buffer of its home rank."""
    require_cuda(rows, meta, peer_rows)
    check(
        lib.xma_b200_ep_return(ptr(rows), dtype_code(rows.dtype), _row_stride(rows), ptr(meta), rows.size(0),
                               rows.size(1), world, ptr(peer_rows), peer_rows_cap, ptr(status_word(rows.device)),
                               current_stream(rows.device)),
        "xma_b200_ep_return",
    )


@torch.library.custom_op(f"{_NS}::swiglu_fwd", mutates_args={"y"}, device_types="cuda")
def _swiglu_fwd_op(g: Tensor, u: Tensor, y: Tensor) -> None:
    require_cuda(g, u, y)
    check(
        lib.xma_b200_swiglu_fwd(
            ptr(g), _row_stride(g), ptr(u), _row_stride(u), ptr(y), _row_stride(y), dtype_code(g.dtype), g.size(0),
            g.size(1), current_stream(g.device)
        ),
        "xma_b200_swiglu_fwd",
    )


@torch.library.custom_op(f"{_NS}::swiglu_bwd", mutates_args={"dg", "du"}, device_types="cuda")
def _swiglu_bwd_op(g: Tensor, u: Tensor, dy: Tensor, dg: Tensor, du: Tensor) -> None:
    require_cuda(g, u, dy, dg, du)
    check(
        lib.xma_b200_swiglu_bwd(
            ptr(g), _row_stride(g), ptr(u), _row_stride(u), ptr(dy), _row_stride(dy), ptr(dg), _row_stride(dg),
            ptr(du), _row_stride(du), dtype_code(g.dtype), g.size(0), g.size(1), current_stream(g.device)
        ),
        "xma_b200_swiglu_bwd",
    )


@torch.library.custom_op(f"{_NS}::swiglu_packed_fwd", mutates_args={"y"}, device_types="cuda")
def _swiglu_packed_fwd_op(x: Tensor, y: Tensor) -> None:
    require_cuda(x, y)
    check(
        lib.xma_b200_swiglu_packed_fwd(
            ptr(x), _row_stride(x), ptr(y), _row_stride(y), dtype_code(x.dtype), y.size(0), y.size(1),
            current_stream(x.device)
        ),
        "xma_b200_swiglu_packed_fwd",
    )


@torch.library.custom_op(f"{_NS}::swiglu_packed_bwd", mutates_args={"dx"}, device_types="cuda")
def _swiglu_packed_bwd_op(x: Tensor, dy: Tensor, dx: Tensor) -> None:
    require_cuda(x, dy, dx)
    check(
        lib.xma_b200_swiglu_packed_bwd(
            ptr(x), _row_stride(x), ptr(dy), _row_stride(dy), ptr(dx), _row_stride(dx), dtype_code(x.dtype),
            dy.size(0), dy.size(1), current_stream(x.device)
        ),
        "xma_b200_swiglu_packed_bwd",
    )


@torch.library.custom_op(f"{_NS}::rmsnorm_fwd", mutates_args={"y", "xr", "rstd"}, device_types="cuda")
def _rmsnorm_fwd_op(x: Tensor, residual: Optional[Tensor], weight: Optional[Tensor], y: Tensor, xr: Optional[Tensor],
                    rstd: Optional[Tensor], eps: float, multiplier: float) -> None:
    require_cuda(x, residual, weight, y, xr, rstd)
    check(
        lib.xma_b200_rmsnorm_fwd(
            ptr(x), _row_stride(x), ptr(residual), 0 if residual is None else _row_stride(residual), ptr(weight),
            ptr(y), _row_stride(y), ptr(xr), 0 if xr is None else _row_stride(xr), ptr(rstd), dtype_code(x.dtype),
            x.size(0), x.size(1), eps, multiplier, current_stream(x.device)
        ),
        "xma_b200_rmsnorm_fwd",
    )


@torch.library.custom_op(f"{_NS}::rmsnorm_bwd", mutates_args={"dx", "dr", "dw_partial"}, device_types="cuda")
def _rmsnorm_bwd_op(xr: Tensor, weight: Optional[Tensor], dy: Tensor, dxr: Optional[Tensor], rstd: Optional[Tensor],
                    dx: Tensor, dr: Optional[Tensor], dw_partial: Optional[Tensor], eps: float,
                    multiplier: float) -> None:
    require_cuda(xr, weight, dy, dxr, rstd, dx, dr, dw_partial)
    check(
        lib.xma_b200_rmsnorm_bwd(
            ptr(xr), _row_stride(xr), ptr(weight), ptr(dy), _row_stride(dy), ptr(dxr),
            0 if dxr is None else _row_stride(dxr), ptr(rstd), ptr(dx), _row_stride(dx), ptr(dr),
            0 if dr is None else _row_stride(dr), ptr(dw_partial), 0 if dw_partial is None else dw_partial.size(0),
            dtype_code(xr.dtype), xr.size(0), xr.size(1), eps, multiplier, current_stream(xr.device)
        ),
        "xma_b200_rmsnorm_bwd",
    )


@torch.library.custom_op(f"{_NS}::router_prob_sums", mutates_args={"partial"}, device_types="cuda")
def _router_prob_sums_op(logits: Tensor, partial: Tensor) -> None:
    require_cuda(logits, partial)
    check(
        lib.xma_b200_router_prob_sums(
            ptr(logits), dtype_code(logits.dtype), _row_stride(logits), logits.size(0), logits.size(1), ptr(partial),
            partial.size(0), current_stream(logits.device)
        ),
        "xma_b200_router_prob_sums",
    )


@torch.library.custom_op(f"{_NS}::load_balancing_loss_bwd", mutates_args={"d_logits"}, device_types="cuda")
def _load_balancing_loss_bwd_op(logits: Tensor, coef: Tensor, d_logits: Tensor) -> None:
    require_cuda(logits, coef, d_logits)
    check(
        lib.xma_b200_load_balancing_loss_bwd(
            ptr(logits), dtype_code(logits.dtype), _row_stride(logits), logits.size(0), logits.size(1), ptr(coef),
            ptr(d_logits), current_stream(logits.device)
        ),
        "xma_b200_load_balancing_loss_bwd",
    )


def _offsets_code(cu_seqlens: Tensor) -> int:
    # uint32 offsets (the reference's tests pass them) read as int32 below 2^31
    if cu_seqlens.dtype in (torch.int32, torch.uint32):
        return _lib.I32
    if cu_seqlens.dtype == torch.int64:
        return _lib.I64
    raise TypeError(f"cu_seqlens must be int32, uint32 or int64, not {cu_seqlens.dtype}")


def _sequence_packing(fn_name: str, src: Tensor, dst: Tensor, padded: Tensor, packed: Tensor, cu_seqlens: Tensor,
                      left: bool) -> None:
    require_cuda(src, dst, cu_seqlens)
    if not (src.is_contiguous() and dst.is_contiguous() and cu_seqlens.is_contiguous()):
        raise ValueError("pack/unpack_sequence kernels take contiguous buffers")
    batch, seq_len = padded.size(0), padded.size(1)
    row = 1
    for d in packed.shape[1:]:
        row *= d
    if tuple(padded.shape[2:]) != tuple(packed.shape[1:]) or cu_seqlens.numel() != batch + 1:
        raise ValueError("padded must be [B, S, ...], packed [T, ...] with the same trailing shape, cu_seqlens [B + 1]")
    check(
        getattr(lib, fn_name)(
            ptr(src), ptr(dst), ptr(cu_seqlens), _offsets_code(cu_seqlens), batch, seq_len, packed.size(0),
            row * packed.element_size(), 1 if left else 0, ptr(status_word(src.device)), current_stream(src.device)
        ),
        fn_name,
    )


@torch.library.custom_op(f"{_NS}::pack_sequence", mutates_args={"packed"}, device_types="cuda")
def _pack_sequence_op(padded: Tensor, cu_seqlens: Tensor, packed: Tensor, left: bool) -> None:
    _sequence_packing("xma_b200_pack_sequence", padded, packed, padded, packed, cu_seqlens, left)


@torch.library.custom_op(f"{_NS}::unpack_sequence", mutates_args={"padded"}, device_types="cuda")
def _unpack_sequence_op(packed: Tensor, cu_seqlens: Tensor, padded: Tensor, left: bool) -> None:
    _sequence_packing("xma_b200_unpack_sequence", packed, padded, padded, packed, cu_seqlens, left)


# ---- launch accounting and per-kernel timing ------------------------------------------------------
class KernelStats:
    """Counts the kernels this library launches and, when `timing` is on, brackets every op with
    CUDA events on the launching stream (used by bench.py for the per-kernel roofline)."""

    def __init__(self) -> None:
        self.enabled = False
        self.timing = False
        self.launches = 0
        self.events: dict[str, list] = {}

    def reset(self) -> None:
        self.launches = 0
        self.events = {}

    def elapsed_ms(self) -> dict[str, list[float]]:
        return {k: [a.elapsed_time(b) for a, b in v] for k, v in self.events.items()}


STATS = KernelStats()


def _wrap(op, name: str, kernels):
    """`kernels`: how many kernels one call launches (an int, or a function of the call's arguments)."""

    def call(*args, tag: str | None = None):
        if not STATS.enabled:
            return op(*args)
        STATS.launches += kernels(*args) if callable(kernels) else kernels
        if not STATS.timing:
            return op(*args)
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        op(*args)
        end.record()
        STATS.events.setdefault(tag or name, []).append((start, end))
        return None

    call.__name__ = name
    return call


continuous_count_ = _wrap(_continuous_count_op, "continuous_count", 1)
route_topk_softmax_ = _wrap(_route_topk_softmax_op, "route_topk_softmax", 1)
route_topk_softmax_bwd_ = _wrap(_route_topk_softmax_bwd_op, "route_topk_softmax_bwd", 1)
count_sort_ = _wrap(_count_sort_op, "count_sort", 4)
gather_rows_ = _wrap(_gather_rows_op, "gather_rows", 1)
spread_rows_ = _wrap(_spread_rows_op, "spread_rows", 1)
combine_rows_ = _wrap(_combine_rows_op, "combine_rows", 1)
combine_bwd_ = _wrap(_combine_bwd_op, "combine_bwd", 1)
def _rows_gemm_kernels(a, w, w_layout, out, aux, row_map, tile_expert, tile_prefix, kd, n, epilogue, impl,
                       out_peers=None, peer_rows_cap=0) -> int:
    """The automatic choice runs a rows GEMM of large experts as two launches: the CTA-pair kernel on the whole
    pairs of 128-row tiles and the one-CTA kernel on the odd last tiles (with up to 16 experts; not when the rows go
    to other ranks; XMA_B200_ODD_TAIL = 0 never, 2 for any number of experts)."""
    split = os.environ.get("XMA_B200_ODD_TAIL", "1")
    if impl != _lib.IMPL_AUTO or out_peers is not None or split == "0" or (split == "1" and w.size(0) > 16):
        return 1
    choice = lib.xma_b200_grouped_gemm_choice(0, dtype_code(a.dtype), w.size(0), tile_expert.numel(), kd, n, w_layout,
                                              epilogue, 0)
    return 2 if choice == _lib.IMPL_TC_PAIR else 1


grouped_gemm_rows_ = _wrap(_grouped_gemm_rows_op, "grouped_gemm_rows", _rows_gemm_kernels)
grouped_gemm_dw_ = _wrap(_grouped_gemm_dw_op, "grouped_gemm_dw", 1)
ep_plan_ = _wrap(_ep_plan_op, "ep_plan", 1)
ep_dispatch_ = _wrap(_ep_dispatch_op, "ep_dispatch", 1)
ep_copy_rows_ = _wrap(_ep_copy_rows_op, "ep_copy_rows", 1)
ep_return_ = _wrap(_ep_return_op, "ep_return", 1)
swiglu_fwd_ = _wrap(_swiglu_fwd_op, "swiglu_fwd", 1)
swiglu_bwd_ = _wrap(_swiglu_bwd_op, "swiglu_bwd", 1)
swiglu_packed_fwd_ = _wrap(_swiglu_packed_fwd_op, "swiglu_packed_fwd", 1)
swiglu_packed_bwd_ = _wrap(_swiglu_packed_bwd_op, "swiglu_packed_bwd", 1)
rmsnorm_fwd_ = _wrap(_rmsnorm_fwd_op, "rmsnorm_fwd", 1)
rmsnorm_bwd_ = _wrap(_rmsnorm_bwd_op, "rmsnorm_bwd", 1)
router_prob_sums_ = _wrap(_router_prob_sums_op, "router_prob_sums", 1)
load_balancing_loss_bwd_ = _wrap(_load_balancing_loss_bwd_op, "load_balancing_loss_bwd", 1)
pack_sequence_ = _wrap(_pack_sequence_op, "pack_sequence", 1)
unpack_sequence_ = _wrap(_unpack_sequence_op, "unpack_sequence", 1)


# Kernel-family override for the grouped GEMMs (tests, tuning): 0 automatic, 1 CUDA cores,
# 2 tcgen05 one CTA per tile, 3 tcgen05 CTA pairs. XMA_B200_GEMM_IMPL sets the initial value.
GEMM_IMPL = int(os.environ.get("XMA_B200_GEMM_IMPL", _lib.IMPL_AUTO))


def set_gemm_impl(impl: int) -> int:
    global GEMM_IMPL
    previous = GEMM_IMPL
    GEMM_IMPL = int(impl)
    return previous
