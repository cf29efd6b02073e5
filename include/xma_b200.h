/*
 * xma_b200.h - C ABI of libxma_b200.so: the MoE hot path of XMA
 * (open-lm-engine/accelerated-model-architectures) as hand-written sm_100a CUDA.
 *
 * Conventions
 *   - Plain pointers and sizes only; every pointer is a DEVICE pointer unless stated otherwise.
 *   - The caller owns and allocates every buffer (outputs included); no entry point allocates device
 *     memory except xma_b200_exchange_alloc (memory that other processes map must not come from a
 *     sub-allocating pool). All work is enqueued on `stream` and is asynchronous.
 *   - Return value: 0 = enqueued; < 0 = argument error found on the host, nothing enqueued
 *     (XMA_ERR_* below); > 0 = cudaError_t of a failed runtime call or launch.
 *     xma_b200_error_string() turns any of them into text.
 *   - `device_status` (may be NULL) is an int32 in device memory that kernels OR bits into:
 *       1 = an id outside [0, bins) was skipped, 2 = a bounded device-side wait expired,
 *       4 = an inconsistent tile table entry was skipped. The caller clears and polls it.
 *   - dtype codes: 0 = fp32, 1 = fp16, 2 = bf16, 3 = int32, 4 = int64.
 *   - Strides are in ELEMENTS. "grouped" buffers hold the routed rows sorted by expert, each
 *     expert's block padded to a multiple of 128 rows (pad rows are zero / ignored).
 *
 * Each entry point names the reference interface (file:line inside the XMA repository) it replaces.
 */
#ifndef XMA_B200_H_
#define XMA_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#ifndef __CUDA_RUNTIME_H__
typedef struct CUstream_st* cudaStream_t;
#endif

#define XMA_B200_ROW_PAD 128

int xma_b200_abi_version(void);
const char* xma_b200_error_string(int code);

/* ---- routing -------------------------------------------------------------------------------- */

/* counts[b] = number of ids equal to b, for b in [0, bins); ids outside the range are skipped
 * (status bit 1). `counts` is overwritten (no pre-zeroing needed).
 * Replaces continuous_count / _continuous_count_cuda:
 *   xma/functional/continuous_count/__init__.py:16-51,
 *   xma/functional/continuous_count/cuda_implementation.py:19-197. */
int xma_b200_continuous_count(const void* ids, int id_dtype, int64_t n, int bins, uint32_t* counts,
                              int* device_status, cudaStream_t stream);

/* logits [tokens, num_experts] (row stride given) -> weights [tokens, top_k] (same dtype as the
 * logits: softmax in fp32 over the top_k selected values, rounded once) and the selected expert
 * ids in descending-logit order (ties: lowest expert id first; NaN sorts above everything).
 * Either index output may be NULL.
 * Replaces MoE._compute_routing_weights after the gate projection and MoE._get_topk:
 *   xma/layers/moe/__init__.py:182-195, 256-262. */
int xma_b200_route_topk_softmax(const void* logits, int dtype, int64_t logits_row_stride, int64_t tokens,
                                int num_experts, int top_k, void* weights, int32_t* selected_i32,
                                int64_t* selected_i64, cudaStream_t stream);

/* d_logits [tokens, num_experts] (dense, fully written) from d_weights [tokens, top_k]: the
 * backward of softmax-over-top-k scattered to the selected columns. The reference gets this from
 * autograd through F.softmax and Tensor.topk (xma/layers/moe/__init__.py:192, 260). */
int xma_b200_route_topk_softmax_bwd(const void* logits, int dtype, int64_t logits_row_stride,
                                    const int32_t* selected_i32, const void* d_weights, int64_t tokens,
                                    int num_experts, int top_k, void* d_logits, cudaStream_t stream);

/* Sizes of the tables and scratch that xma_b200_count_sort needs for n routed ids and E experts. */
int64_t xma_b200_count_sort_scratch_bytes(int64_t n, int num_experts);
int64_t xma_b200_tile_capacity(int64_t n, int num_experts); /* 128-row tiles: n / 128 + E */

/* Stable counting sort of the n routed expert ids (id i belongs to flat index i = token*top_k+slot):
 *   counts[E]                 rows per expert (== bincount)
 *   offsets_incl[E]           inclusive prefix sum of counts
 *   pad_offsets[E+1]          first row of each expert in the padded grouped layout
 *   tile_prefix[E+1]          128-row tiles in front of each expert; [E] = tiles in use
 *   tile_expert[tile_cap]     owner of each padded tile
 *   sorted_expert_idxs[n]     ids ascending
 *   sorted_scattered_idxs[n]  flat index of each sorted row (stable: ties by flat index)
 *   row_src[row_cap]          flat index of each PADDED grouped row, -1 for pad rows (may be NULL)
 *   row_dst[n]                the inverse map: padded grouped row of each flat index, -1 for an id
 *                             out of range (may be NULL)
 * tile_cap >= xma_b200_tile_capacity(n, E); row_cap >= 128 * tile_cap; scratch is 256-byte
 * aligned, scratch_bytes >= xma_b200_count_sort_scratch_bytes(n, E); num_experts <= 1024.
 * Replaces `selected_experts.flatten().sort()`, continuous_count and cumsum in
 *   xma/layers/moe/__init__.py:210-217. */
int xma_b200_count_sort(const void* ids, int id_dtype, int64_t n, int num_experts, uint32_t* counts,
                        int32_t* offsets_incl, int32_t* pad_offsets, int32_t* tile_prefix, int32_t* tile_expert,
                        int64_t tile_cap, int32_t* sorted_expert_idxs, int32_t* sorted_scattered_idxs,
                        int32_t* row_src, int64_t row_cap, int32_t* row_dst, void* scratch, int64_t scratch_bytes,
                        int* device_status, cudaStream_t stream);

/* xma_b200_count_sort for callers that may not allocate device memory while they run (an engine
 * that gave its whole budget to a pool at start-up, a step wedged between other allocators): the
 * scratch comes from a fixed array inside the library (held by every GPU that loads it, until
 * exit) instead of a caller buffer, and nothing is allocated or freed. Outputs are identical to
 * xma_b200_count_sort. Limits: the scratch the problem needs
 * (xma_b200_count_sort_scratch_bytes) must not exceed
 * xma_b200_count_sort_static_scratch_limit() = 524544 bytes, e.g. up to 2 Mi ids with 256
 * experts, else XMA_ERR_TOO_LARGE (-8). The first call on a device resolves the array's device
 * address; issue it before any stream capture, and at start-up: under lazy module loading it may be
 * the moment the driver places the library's code and the array on the device (a driver-side
 * allocation), which should happen before a memory pool takes the budget. Calls on one device share
 * the array (cleared at the start of each call); calls that overlap on the GPU race.
 * This entry point has no counterpart in the reference. */
int64_t xma_b200_count_sort_static_scratch_limit(void);
int xma_b200_count_sort_static(const void* ids, int id_dtype, int64_t n, int num_experts, uint32_t* counts,
                               int32_t* offsets_incl, int32_t* pad_offsets, int32_t* tile_prefix,
                               int32_t* tile_expert, int64_t tile_cap, int32_t* sorted_expert_idxs,
                               int32_t* sorted_scattered_idxs, int32_t* row_src, int64_t row_cap,
                               int* device_status, cudaStream_t stream);

/* ---- row movement --------------------------------------------------------------------------- */

/* out[p, :] = src[row_src[p] / fan_out, :] * coeff[row_src[p]]  (coeff may be NULL; rows with
 * row_src[p] < 0 are written as zeros). Only the first *rows_in_use rows are touched when that
 * device pointer is non-NULL. width and strides must keep rows 16-byte aligned.
 * Replaces group: xma/layers/moe/triton_implementation/group_kernel.py:69-100. */
int xma_b200_gather_rows(const void* src, int dtype, int64_t src_row_stride, const int32_t* row_src,
                         const void* coeff, int fan_out, int64_t rows, const int32_t* rows_in_use, int64_t width,
                         void* out, int64_t out_row_stride, cudaStream_t stream);

/* Token-major form of xma_b200_gather_rows for the routed rows (row_dst from xma_b200_count_sort): for every
 * token t and slot k < top_k
 *   out[row_dst[t * top_k + k], :] = src[t, :] * coeff[t * top_k + k]     (coeff NULL: 1; row_dst < 0: skipped)
 * and every expert's pad rows [pad_offsets[e] + counts[e], pad_offsets[e + 1]) of `out` are written as zeros.
 * With ys / d_weights (both or neither): d_weights[t * top_k + k] = <ys[t * top_k + k, :], src[t, :]>, which is
 * xma_b200_combine_bwd on the row that is in registers anyway. A token's row is read once instead of once per
 * slot. top_k <= 32. Replaces group (group_kernel.py:69-100) and, fused, the bmm of
 * xma/layers/moe/triton_implementation/__init__.py:130-131. */
int xma_b200_spread_rows(const void* src, int dtype, int64_t src_row_stride, const int32_t* row_dst, const void* coeff,
                         const void* ys, int64_t ys_row_stride, void* d_weights, int top_k, int64_t tokens,
                         int64_t width, void* out, int64_t out_row_stride, const uint32_t* counts,
                         const int32_t* pad_offsets, int num_experts, cudaStream_t stream);

/* y[t, :] = sum_k weights[t, k] * ys[row(t * top_k + k), :], fp32 accumulate, one rounding
 * (weights NULL: plain sum over the top_k slots). row(f) = row_index[f] when row_index is given
 * (ys kept in another row order, e.g. expert-sorted), f otherwise.
 * Replaces the bmm combine and the K-slot sum:
 *   xma/layers/moe/triton_implementation/__init__.py:100-101 and :70. */
int xma_b200_combine_rows(const void* ys, int dtype, int64_t ys_row_stride, const void* weights,
                          const int32_t* row_index, int top_k, int64_t tokens, int64_t width, void* y,
                          int64_t y_row_stride, cudaStream_t stream);

/* d_weights[t, k] = <ys[row(t * top_k + k), :], dy[t, :]>.
 * Replaces the bmm of xma/layers/moe/triton_implementation/__init__.py:130-131. */
int xma_b200_combine_bwd(const void* ys, int dtype, int64_t ys_row_stride, const void* dy, int64_t dy_row_stride,
                         const int32_t* row_index, int top_k, int64_t tokens, int64_t width, void* d_weights,
                         cudaStream_t stream);

/* ---- expert grouped GEMMs ------------------------------------------------------------------- */

/* w_layout: 0 = weight stored [E, n, kd] (out = a * w_e^T), 1 = weight stored [E, kd, n] (out = a * w_e).
 * epilogue: 0 = plain store (rows optionally scattered through row_map, negative entries skipped);
 *           1 = SwiGLU forward, n = 2I: aux[r, 0:2I] = gate|up (rounded), out[r, 0:I] = up*gate*sigmoid(gate);
 *           2 = SwiGLU backward, n = I: aux holds gate|up, the contraction is d(activation),
 *               out[r, 0:I] = d gate, out[r, I:2I] = d up.
 *           3 / 4 = the same two with gate and up interleaved along the columns (g,u,g,u,...: the layout of
 *               swiglu_packed); tensor-core kernels only (XMA_ERR_UNSUPPORTED otherwise).
 * impl: 0 = automatic, 1 = CUDA cores, 2 = tcgen05 tensor cores with one CTA per 128x256 tile, 3 = tcgen05
 *       with CTA pairs (cta_group::2, 256x256 tiles); 2 and 3 need bf16/fp16 and widths that are multiples of 8.
 * a is grouped [128 * tile_cap, kd]. fp32 accumulation everywhere.
 * Replaces scatter2scatter: xma/layers/moe/triton_implementation/scatter_kernel.py:137-183,
 * with swiglu fused as in xma/functional/swiglu/__init__.py:39. */
int xma_b200_grouped_gemm_rows(const void* a, int64_t a_row_stride, const void* w, int w_layout, void* out,
                               int64_t out_row_stride, void* aux, int64_t aux_row_stride, const int32_t* row_map,
                               const int32_t* tile_expert, const int32_t* tile_prefix, int num_experts,
                               int64_t tile_cap, int64_t kd, int64_t n, int epilogue, int dtype, int impl,
                               int* device_status, cudaStream_t stream);

/* The same GEMM with its output rows stored into other ranks' memory (expert parallelism): plain
 * epilogue and row_map required; row_map[r] = (rank << 24) | row (negative: skipped) and the row is
 * stored to out_peers[rank] + row * out_row_stride, where out_peers is a device table of one base
 * address per rank (this rank's own buffer included; the others mapped with xma_b200_exchange_open).
 * out_peers has peer_world entries (<= 128) and every rank's buffer peer_rows_cap rows (<= 2^24): a
 * word that names a rank or a row outside them is skipped like a negative one and sets status bit 1,
 * so a stale or corrupt word never becomes a store into another GPU's memory.
 * The tensor-core kernels (one CTA per tile and CTA pairs) stage the tile in shared memory so that
 * every row crosses NVLink in 128-byte pieces. out_peers NULL: identical to
 * xma_b200_grouped_gemm_rows (peer_world and peer_rows_cap ignored). No counterpart in the reference,
 * whose MoE keeps all experts on one device (xma/layers/moe/__init__.py:144-160). */
int xma_b200_grouped_gemm_rows_peer(const void* a, int64_t a_row_stride, const void* w, int w_layout, void* out,
                                    int64_t out_row_stride, void* aux, int64_t aux_row_stride,
                                    const int32_t* row_map, void* const* out_peers, int peer_world,
                                    int64_t peer_rows_cap, const int32_t* tile_expert, const int32_t* tile_prefix,
                                    int num_experts, int64_t tile_cap, int64_t kd, int64_t n, int epilogue, int dtype,
                                    int impl, int* device_status, cudaStream_t stream);

/* dw[e, m, n] = sum over the rows r of expert e of x[r, m] * y[r, n]; x, y grouped (rows_cap rows
 * allocated); experts without rows get zeros, so dw needs no pre-zeroing.
 * Replaces group_bwd_W: xma/layers/moe/triton_implementation/group_backward_kernel.py:102-128. */
int xma_b200_grouped_gemm_dw(const void* x, int64_t x_row_stride, const void* y, int64_t y_row_stride,
                             const uint32_t* counts, const int32_t* pad_offsets, int64_t rows_cap, int num_experts,
                             int64_t m, int64_t n, void* dw, int dtype, int impl, int* device_status,
                             cudaStream_t stream);

int xma_b200_grouped_gemm_uses_tensor_cores(int dtype, int64_t kd, int64_t n);

/* Host-only query: the kernel family that impl = 0 takes on the current device for a problem of this
 * shape, assuming 16-byte aligned pointers (1 = CUDA cores, 2 = tcgen05 one CTA per tile, 3 = tcgen05
 * CTA pairs). kind 0 = xma_b200_grouped_gemm_rows(_peer) with kd, n, w_layout, epilogue and peer
 * (0/1: out_peers given); kind 1 = xma_b200_grouped_gemm_dw with m = kd, n. No counterpart in the
 * reference (its Triton autotuner picks tile sizes, xma/layers/moe/triton_implementation/scatter_kernel.py:12-52). */
int xma_b200_grouped_gemm_choice(int kind, int dtype, int num_experts, int64_t tile_cap, int64_t kd, int64_t n,
                                 int w_layout, int epilogue, int peer);

/* Process-wide tuning switches of the tensor-core kernels; returns the previous value (< 0: unknown key).
 * key 0: SwiGLU-backward epilogue asks for the next tile's gate|up rows in L2 (0/1, default 1);
 * key 1: reduction blocks that the TMA producer prefetches into L2 ahead of its loads (0..255, default 0);
 * key 2: operands that prefetch covers (bit 0 = A, bit 1 = B); key 3: epilogue warps (0 = per-kernel
 * default, 4, 8); key 4: CTA pairs also for plain epilogues in the automatic choice (0/1, default 1);
 * key 5: the CTA-pair weight-gradient kernel hands its tiles out by an atomic ticket, heaviest experts first,
 * instead of a fixed stride (0/1, default 1);
 * key 6: the SwiGLU epilogues of the CTA-pair kernel move their tiles through shared memory by TMA, 32 columns at a
 * time, instead of reading and writing them with one row per thread, when the activation width is a multiple of 32
 * and there are at most 192 experts: bit 0 = backward (gate|up read, d gate|d up written; both layouts), bit 1 = forward
 * (gate|up and the activation written; only for reductions shorter than 4096 unless bit 2 is set); default 3.
 * key 7: with the automatic choice (impl 0) a rows GEMM of large experts runs as two launches, the CTA-pair kernel
 * on the whole pairs of 128-row tiles of every expert and the one-CTA kernel on the last tile of the experts that
 * have an odd number of them (1, the default: with up to 16 experts, where it was measured to pay; 2: with any
 * number), or as one launch of the CTA-pair kernel, which then computes a 256-row tile for an odd last tile (0);
 * rows stored into other ranks' buffers always take one launch.
 * The environment variables XMA_B200_GU_PREFETCH, XMA_B200_TMA_PREFETCH, XMA_B200_TMA_PREFETCH_MASK,
 * XMA_B200_EPI_WARPS, XMA_B200_PLAIN_PAIRS, XMA_B200_DW_DYNAMIC, XMA_B200_DSWIGLU_STAGED and XMA_B200_ODD_TAIL set
 * the initial values.
 * Stands where the reference has its autotune configurations (scatter_kernel.py:12-52). */
int xma_b200_tuning_set(int key, int value);

/* ---- stand-alone SwiGLU --------------------------------------------------------------------- */

/* y = up * gate * sigmoid(gate) in fp32, rounded once; row-strided operands allowed.
 * Replaces _swiglu_forward_cuda / _swiglu_backward_cuda and the packed variants:
 *   xma/functional/swiglu/__init__.py:39-87,
 *   xma/functional/swiglu/cuda_implementation/__init__.py:13-63. */
int xma_b200_swiglu_fwd(const void* gate, int64_t gate_row_stride, const void* up, int64_t up_row_stride, void* y,
                        int64_t y_row_stride, int dtype, int64_t rows, int64_t cols, cudaStream_t stream);
int xma_b200_swiglu_bwd(const void* gate, int64_t gate_row_stride, const void* up, int64_t up_row_stride,
                        const void* dy, int64_t dy_row_stride, void* dgate, int64_t dgate_row_stride, void* dup,
                        int64_t dup_row_stride, int dtype, int64_t rows, int64_t cols, cudaStream_t stream);
/* x[r, 2c] = gate, x[r, 2c + 1] = up; out_cols is the width of y (half the width of x). */
int xma_b200_swiglu_packed_fwd(const void* x, int64_t x_row_stride, void* y, int64_t y_row_stride, int dtype,
                               int64_t rows, int64_t out_cols, cudaStream_t stream);
int xma_b200_swiglu_packed_bwd(const void* x, int64_t x_row_stride, const void* dy, int64_t dy_row_stride,
                               void* dx, int64_t dx_row_stride, int dtype, int64_t rows, int64_t out_cols,
                               cudaStream_t stream);

/* ---- fused residual add + RMSNorm (the step in front of the MoE layer) ----------------------- */

/* v = x * multiplier + residual (residual NULL: v = x * multiplier), rounded to the storage type;
 * xr = v (written when xr != NULL; required when residual != NULL); rstd[r] = rsqrt(mean(v[r]^2) + eps)
 * (written when rstd != NULL); y = v * rstd * weight (weight NULL: 1). fp32 arithmetic, one rounding per output.
 * Replaces fused_residual_add_rmsnorm and its Triton forward:
 *   xma/functional/fused_residual_add_rmsnorm/__init__.py:27-83, template.py:12-34,
 *   triton_implementation/forward.py. */
int xma_b200_rmsnorm_fwd(const void* x, int64_t x_row_stride, const void* residual, int64_t residual_row_stride,
                         const void* weight, void* y, int64_t y_row_stride, void* xr, int64_t xr_row_stride,
                         float* rstd, int dtype, int64_t rows, int64_t cols, float eps, float multiplier,
                         cudaStream_t stream);
/* Backward of the above, given xr (the value the norm saw), dy and optionally d(xr) (gradient that arrives
 * through the residual stream) and rstd (NULL: recomputed from xr):
 *   z = xr * rstd, g = dy * weight, d = (g - z * mean(g * z)) * rstd + dxr;  dresidual = d (when != NULL),
 *   dx = d * multiplier,  dweight_partial[b, :] = sum over the rows CTA b handled of dy * z  (fp32,
 *   [partial_rows, cols] with partial_rows = xma_b200_rmsnorm_bwd_partial_rows(rows); the caller sums over b).
 * Replaces template.py:37-84 and triton_implementation/backward.py:15-150 (same partial-sum scheme). */
int xma_b200_rmsnorm_bwd_partial_rows(int64_t rows);
int xma_b200_rmsnorm_bwd(const void* xr, int64_t xr_row_stride, const void* weight, const void* dy,
                         int64_t dy_row_stride, const void* dxr, int64_t dxr_row_stride, const float* rstd, void* dx,
                         int64_t dx_row_stride, void* dresidual, int64_t dresidual_row_stride, float* dweight_partial,
                         int partial_rows, int dtype, int64_t rows, int64_t cols, float eps, float multiplier,
                         cudaStream_t stream);

/* ---- auxiliary load-balancing loss on the router logits --------------------------------------- */
/* No counterpart in the reference, which returns router_logits unused (xma/layers/moe/__init__.py:180); this is the
 * usual consumer: loss = E * sum_e f_e * P_e with P_e = mean over tokens of softmax(logits)[t, e] (fp32) and
 * f_e = (routed slots of expert e) / tokens, a count without gradient (Switch Transformer, eq. 4-6).
 * _sums: partial[b, e] = sum over the tokens CTA b handled of softmax(logits[t, :])[e], b < partial_rows =
 * xma_b200_router_prob_partial_rows(tokens) (fp32 [partial_rows, E]; the caller adds the rows up, a fixed order).
 * _bwd: d_logits[t, j] = p[t, j] * (coef[j] - sum_e coef[e] * p[t, e]) with coef[e] = d loss * E * f_e / tokens
 * (fp32 [E], device); d_logits is dense [tokens, E] in the dtype of the logits. num_experts <= 1024. */
int xma_b200_router_prob_partial_rows(int64_t tokens);
int xma_b200_router_prob_sums(const void* logits, int dtype, int64_t logits_row_stride, int64_t tokens,
                              int num_experts, float* partial, int partial_rows, cudaStream_t stream);
int xma_b200_load_balancing_loss_bwd(const void* logits, int dtype, int64_t logits_row_stride, int64_t tokens,
                                     int num_experts, const float* coef, void* d_logits, cudaStream_t stream);

/* ---- pack_sequence / unpack_sequence ----------------------------------------------------------- */
/* Replace the kernels behind xma.functional.pack_sequence / unpack_sequence
 * (xma/functional/sequence_packing/__init__.py:39-132; cuda_implementation.py:17-98, launched from :101-134;
 * semantics of torch_implementation.py:9-48).
 *   padded [batch, seq_len, row]   packed [total_tokens, row]   cu_seqlens [batch + 1] (device; cu_dtype XMA_I32 -
 *   which also takes uint32 offsets below 2^31 - or XMA_I64), row given in BYTES (product of the trailing
 *   dimensions x itemsize): the kernels copy bytes and do not care about the element type.
 * Sequence b holds tokens cu_seqlens[b] .. cu_seqlens[b + 1] - 1 of the packed buffer; in the padded buffer they
 * are the LAST len_b positions of row b (left_padding != 0) or the first (left_padding == 0).
 * _pack: writes every row of `packed`: the tokens of the sequences (cu_seqlens[0] = 0) and zeros in rows behind
 * cu_seqlens[batch], if total_tokens is larger.
 * _unpack: writes ALL of `padded`, the tokens and zeros in the padding (no zero-fill by the caller).
 * A sequence whose offsets leave [0, total_tokens] or whose length exceeds seq_len is skipped (zeros on unpack) and
 * sets bit 1 of *device_status (may be NULL). Both buffers contiguous; any alignment (the copy unit adapts). */
int xma_b200_pack_sequence(const void* padded, void* packed, const void* cu_seqlens, int cu_dtype, int64_t batch,
                           int64_t seq_len, int64_t total_tokens, int64_t row_bytes, int left_padding,
                           int* device_status, cudaStream_t stream);
int xma_b200_unpack_sequence(const void* packed, void* padded, const void* cu_seqlens, int cu_dtype, int64_t batch,
                             int64_t seq_len, int64_t total_tokens, int64_t row_bytes, int left_padding,
                             int* device_status, cudaStream_t stream);

/* ---- expert parallelism over peer memory ------------------------------------------------------ */
/* None of these has a counterpart in the reference (single-device MoE, xma/layers/moe/__init__.py:144-160).
 * Rank r of `world` owns experts [r * E / world, (r + 1) * E / world). An owner keeps the rows it receives
 * expert-major, inside an expert ordered by source rank, every expert padded to 128 rows. No kernel waits
 * on another GPU: the caller separates the phases with a stream-ordered barrier over all ranks. */

/* count_matrix [world, E] (int32, device): rows rank s routes to global expert e. Writes, for this rank:
 * send_delta [E] (sorted row p of expert e lands in row p + send_delta[e] of the owner's buffer), and the
 * grouped layout of its own E / world experts (counts, pad_offsets [E/world + 1], tile_prefix [E/world + 1],
 * tile_expert [tile_cap]); resets the pad slots of `meta` (this rank's origin words, meta_cap entries) to -1.
 * Sets device status bit 4 and an empty layout if tile_cap or meta_cap is too small. */
int xma_b200_ep_plan(const int32_t* count_matrix, int world, int num_experts, int rank, int32_t* send_delta,
                     uint32_t* counts, int32_t* pad_offsets, int32_t* tile_prefix, int32_t* tile_expert,
                     int64_t tile_cap, int32_t* meta, int64_t meta_cap, int* device_status, cudaStream_t stream);

/* Dispatch: for every sorted row p (q = sorted_scattered_idxs[p], e = sorted_expert_idxs[p], owner = e / (E/world))
 *   peer_rows[owner][p + send_delta[e], :] = src[q / fan_out, :] * coeff[q]   (coeff NULL: 1)
 *   peer_meta[owner][p + send_delta[e]]    = (rank << 24) | q                 (peer_meta NULL: not written)
 * peer_rows / peer_meta: device tables of one base address per rank; rows of `width` elements, dense.
 * Rows that would fall outside [0, peer_rows_cap) are not stored and set device status bit 1. */
int xma_b200_ep_dispatch(const void* src, int dtype, int64_t src_row_stride, const int32_t* sorted_expert_idxs,
                         const int32_t* sorted_scattered_idxs, const void* coeff, int fan_out,
                         const int32_t* send_delta, int num_experts, int world, int rank, int64_t rows, int64_t width,
                         void* const* peer_rows, int32_t* const* peer_meta, int64_t peer_rows_cap,
                         int* device_status, cudaStream_t stream);

/* The same for the rows of this rank whose expert is one of the owners' local experts [local_lo, local_hi) only
 * (local index = e mod (E / world)): the exchange cut into parts by expert, so that the owners can start on the
 * experts of one part while the rows of the next are still on their way. */
int xma_b200_ep_dispatch_part(const void* src, int dtype, int64_t src_row_stride, const int32_t* sorted_expert_idxs,
                              const int32_t* sorted_scattered_idxs, const void* coeff, int fan_out,
                              const int32_t* send_delta, int num_experts, int world, int rank, int local_lo,
                              int local_hi, int64_t rows, int64_t width, void* const* peer_rows,
                              int32_t* const* peer_meta, int64_t peer_rows_cap, int* device_status,
                              cudaStream_t stream);

/* out[r, :] = meta[r] >= 0 ? rows[r, :] : 0 for r < n_rows (dense rows of `width` elements);
 * out == rows zero-fills the pad rows in place. */
int xma_b200_ep_copy_rows(const void* rows, int dtype, const int32_t* meta, int64_t n_rows, int64_t width, void* out,
                          cudaStream_t stream);

/* host_words[i] = src[i] for i < n, written by a kernel: host_words is pinned host memory that the device
 * addresses directly (cudaHostAlloc / cudaHostRegister under unified addressing). The host reads it after
 * an event recorded behind the call; unlike a device->host copy it does not wait in the copy engine's queue. */
int xma_b200_ep_publish(const int32_t* src, int64_t n, int32_t* host_words, cudaStream_t stream);

/* Return: peer_rows[meta[r] >> 24][meta[r] & 0xffffff, :] = rows[r, :] for every r < n_rows with meta[r] >= 0
 * (expert output rows back to the token's home rank, whole rows per warp store): the unfused form of what
 * xma_b200_grouped_gemm_rows_peer does in its epilogue. */
int xma_b200_ep_return(const void* rows, int dtype, int64_t row_stride, const int32_t* meta, int64_t n_rows,
                       int64_t width, int world, void* const* peer_rows, int64_t peer_rows_cap, int* device_status,
                       cudaStream_t stream);

/* Exchange buffers: zero-filled device memory of the current device that the other processes of the node map
 * into their address space (CUDA IPC; the devices must be peers). _export writes
 * xma_b200_exchange_handle_bytes() bytes that another process hands to _open; _close unmaps, _free releases. */
int xma_b200_exchange_alloc(int64_t bytes, void** out_ptr);
int xma_b200_exchange_free(void* ptr);
int xma_b200_exchange_handle_bytes(void);
int xma_b200_exchange_export(void* ptr, void* handle_out);
int xma_b200_exchange_open(const void* handle, void** out_ptr);
int xma_b200_exchange_close(void* ptr);

#ifdef __cplusplus
}
#endif

#endif /* XMA_B200_H_ */
