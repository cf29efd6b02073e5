// Expert-parallel row exchange over peer memory (NVLink / NVSwitch), one process per GPU.
//
// The reference keeps every expert on one device (xma/layers/moe/__init__.py:144-160); sharding
// the experts over ranks adds a dispatch (token rows -> the rank that owns their expert) and a
// combine (expert outputs -> the token's home rank). Both are done with plain stores into the
// destination rank's memory, which the host maps into this process once:
//   * ep_plan_kernel     : from the W x E matrix of per-rank expert counts, where each of this
//                          rank's sorted rows lands in its owner's padded expert-major buffer, and
//                          the tile tables of the experts this rank owns.
//   * ep_dispatch_kernel : gather of the routed token rows fused with the exchange - every row is
//                          written straight to (owner, row) together with a word that names its
//                          origin (home rank << 24 | token slot).
//   * ep_copy_rows_kernel: owner side, received rows -> private padded buffer (pad rows zero),
//                          or zero-fill of the pad rows in place.
//   * ep_return_kernel   : owner side, expert output rows -> the home rank named by their origin
//                          word, whole rows at a time (512 contiguous bytes per warp store).
// By default the way back is fused into the grouped GEMM instead (`out_peers` of the rows GEMM): its
// epilogue stores each output row to its home rank. An epilogue thread owns one accumulator row, so
// storing straight from registers would be 32 pieces of 16 bytes in 32 rows per warp instruction,
// which NVLink moved at about 125 GB/s; the epilogue therefore stages 64 columns in shared memory and
// stores 128 contiguous bytes per row, which hides the exchange inside the GEMM (8 GPUs, 128 experts
// top-8: down projection 1.33 ms plain + 1.41 ms return kernel -> 1.54 ms fused).
// No kernel here waits on another GPU; ranks are ordered by the caller's stream-ordered barrier
// between the phases.
#include "common.cuh"

#include <cstring>

namespace xma {

constexpr int EP_PLAN_THREADS = 256;
constexpr int EP_MAX_EXPERTS = 1024;
constexpr int EP_ROW_THREADS = 256;
constexpr int EP_ROWS = 4;  // rows per CTA iteration: that many independent 128-bit loads per thread

// count_matrix[s * E + e] = rows rank s routes to (global) expert e; rank r owns experts
// [r * e_local, (r + 1) * e_local). An owner's buffer is expert-major, inside an expert
// source-rank-major, each expert padded to XMA_ROW_PAD rows.
//   send_delta[e]  : sorted position p of this rank (expert e) -> row p + send_delta[e] at the owner
//   counts/pad_offsets/tile_prefix/tile_expert : the grouped layout of the experts this rank owns
//   meta           : this rank's own origin words; pad slots are reset to -1 here (valid slots are
//                    written by the senders, the two sets are disjoint)
__global__ void __launch_bounds__(EP_PLAN_THREADS)
ep_plan_kernel(const int* __restrict__ count_matrix, int W, int E, int rank, int* __restrict__ send_delta,
               unsigned* __restrict__ counts, int* __restrict__ pad_offsets, int* __restrict__ tile_prefix,
               int* __restrict__ tile_expert, int tile_cap, int* __restrict__ meta, int64_t meta_cap,
               int* __restrict__ status) {
    __shared__ int s_total[EP_MAX_EXPERTS];
    __shared__ int s_before[EP_MAX_EXPERTS];
    __shared__ int s_tiles_total;
    const int e_local = E / W;
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        int total = 0, before = 0;
        for (int s = 0; s < W; ++s) {
            const int c = count_matrix[s * E + e];
            if (s < rank) before += c;
            total += c;
        }
        s_total[e] = total;
        s_before[e] = before;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int my_run = 0;  // exclusive offset of expert e among this rank's sorted rows
        for (int w = 0; w < W; ++w) {
            int pad = 0, tiles = 0;
            for (int j = 0; j < e_local; ++j) {
                const int e = w * e_local + j;
                send_delta[e] = pad + s_before[e] - my_run;
                my_run += count_matrix[rank * E + e];
                const int t = (s_total[e] + XMA_ROW_PAD - 1) / XMA_ROW_PAD;
                if (w == rank) {
                    counts[j] = static_cast<unsigned>(s_total[e]);
                    pad_offsets[j] = pad;
                    tile_prefix[j] = tiles;
                }
                tiles += t;
                pad += t * XMA_ROW_PAD;
            }
            if (w == rank) {
                if (tiles > tile_cap || pad > meta_cap) {  // the host sized both from the same matrix
                    if (status) atomicOr(status, XMA_DEV_BAD_TILE);
                    tiles = 0;
                    pad = 0;
                }
                pad_offsets[e_local] = pad;
                tile_prefix[e_local] = tiles;
                s_tiles_total = tiles;
            }
        }
    }
    __syncthreads();
    const int total_tiles = s_tiles_total;
    for (int j = threadIdx.x; j < e_local; j += blockDim.x) {
        const int c = s_total[rank * e_local + j];
        const int t0 = tile_prefix[j];
        int t1 = t0 + (c + XMA_ROW_PAD - 1) / XMA_ROW_PAD;
        if (t1 > total_tiles) t1 = total_tiles;
        for (int t = t0; t < t1; ++t) tile_expert[t] = j;
        const int r1 = pad_offsets[j] + (t1 - t0) * XMA_ROW_PAD;
        for (int r = pad_offsets[j] + c; r < r1; ++r) meta[r] = -1;
    }
}

// Row p of this rank's expert-sorted order (token slot q = sorted_scattered[p], expert
// e = sorted_expert[p]) goes to rank e / e_local, row p + send_delta[e]:
//   peer_rows[owner][row, :] = src[q / fan_out, :] * coeff[q],   peer_meta[owner][row] = rank << 24 | q
template <typename T, bool HAS_COEFF>
__global__ void __launch_bounds__(EP_ROW_THREADS)
ep_dispatch_kernel(const T* __restrict__ src, int64_t src_stride, const int* __restrict__ sorted_expert,
                   const int* __restrict__ sorted_scattered, const T* __restrict__ coeff, int fan_out,
                   const int* __restrict__ send_delta, int num_experts, int e_local, int local_lo, int local_hi,
                   int rank, int64_t rows, int64_t width, void* const* __restrict__ peer_rows,
                   int* const* __restrict__ peer_meta, int64_t peer_rows_cap, int* __restrict__ status) {
    constexpr int V = Vec16<T>::N;
    const int64_t nvec = width / V;
    for (int64_t p0 = static_cast<int64_t>(blockIdx.x) * EP_ROWS; p0 < rows;
         p0 += static_cast<int64_t>(gridDim.x) * EP_ROWS) {
        int q[EP_ROWS];
        T* dst[EP_ROWS];
        float cf[EP_ROWS];
#pragma unroll
        for (int j = 0; j < EP_ROWS; ++j) {
            q[j] = -1;
            dst[j] = nullptr;
            cf[j] = 1.0f;
            if (p0 + j < rows) {
                const int e = sorted_expert[p0 + j];
                const int qq = sorted_scattered[p0 + j];
                const int64_t row = (e >= 0 && e < num_experts) ? p0 + j + send_delta[e] : -1;
                if (row < 0 || row >= peer_rows_cap || qq < 0 || qq > PEER_ROW_MASK) {
                    if (threadIdx.x == 0 && status) atomicOr(status, XMA_DEV_ID_OUT_OF_RANGE);
                    continue;  // never store outside the owner's buffer
                }
                const int owner = e / e_local;
                const int local = e - owner * e_local;
                if (local < local_lo || local >= local_hi) continue;  // another part of the pipelined exchange
                q[j] = qq;
                dst[j] = static_cast<T*>(peer_rows[owner]) + row * width;
                if (HAS_COEFF) cf[j] = to_f32(coeff[qq]);
                if (threadIdx.x == 0 && peer_meta) peer_meta[owner][row] = (rank << PEER_ROW_BITS) | qq;
            }
        }
        for (int64_t c = threadIdx.x; c < nvec; c += EP_ROW_THREADS) {
            Vec16<T> x[EP_ROWS];
#pragma unroll
            for (int j = 0; j < EP_ROWS; ++j)
                if (q[j] >= 0) x[j] = load16(src + static_cast<int64_t>(q[j] / fan_out) * src_stride + c * V);
#pragma unroll
            for (int j = 0; j < EP_ROWS; ++j) {
                if (q[j] < 0) continue;
                if (HAS_COEFF) {
#pragma unroll
                    for (int i = 0; i < V; ++i) x[j].v[i] = from_f32<T>(to_f32(x[j].v[i]) * cf[j]);
                }
                store16(dst[j] + c * V, x[j]);
            }
        }
    }
}

// out[r, :] = meta[r] >= 0 ? rows[r, :] : 0 for r < n_rows. IN_PLACE: only the pad rows are touched.
template <typename T, bool IN_PLACE>
__global__ void __launch_bounds__(EP_ROW_THREADS)
ep_copy_rows_kernel(const T* __restrict__ rows, const int* __restrict__ meta, int64_t n_rows, int64_t width,
                    T* __restrict__ out) {
    constexpr int V = Vec16<T>::N;
    const int64_t nvec = width / V;
    for (int64_t p0 = static_cast<int64_t>(blockIdx.x) * EP_ROWS; p0 < n_rows;
         p0 += static_cast<int64_t>(gridDim.x) * EP_ROWS) {
        int m[EP_ROWS];
#pragma unroll
        for (int j = 0; j < EP_ROWS; ++j) m[j] = (p0 + j < n_rows) ? (meta[p0 + j] >= 0 ? 1 : 0) : -1;
        if (IN_PLACE && m[0] != 0 && m[1] != 0 && m[2] != 0 && m[3] != 0) continue;
        for (int64_t c = threadIdx.x; c < nvec; c += EP_ROW_THREADS) {
            Vec16<T> x[EP_ROWS];
#pragma unroll
            for (int j = 0; j < EP_ROWS; ++j) {
                if (!IN_PLACE && m[j] == 1) {
                    x[j] = load16_stream(rows + (p0 + j) * width + c * V);
                } else {
#pragma unroll
                    for (int i = 0; i < V; ++i) x[j].v[i] = from_f32<T>(0.0f);
                }
            }
#pragma unroll
            for (int j = 0; j < EP_ROWS; ++j) {
                if (m[j] < 0 || (IN_PLACE && m[j] == 1)) continue;
                store16(out + (p0 + j) * width + c * V, x[j]);
            }
        }
    }
}

// peer_rows[meta[r] >> 24][meta[r] & mask, :] = rows[r, :] for every r < n_rows with meta[r] >= 0.
template <typename T>
__global__ void __launch_bounds__(EP_ROW_THREADS)
ep_return_kernel(const T* __restrict__ rows, int64_t row_stride, const int* __restrict__ meta, int64_t n_rows,
                 int64_t width, int world, void* const* __restrict__ peer_rows, int64_t peer_rows_cap,
                 int* __restrict__ status) {
    constexpr int V = Vec16<T>::N;
    const int64_t nvec = width / V;
    for (int64_t p0 = static_cast<int64_t>(blockIdx.x) * EP_ROWS; p0 < n_rows;
         p0 += static_cast<int64_t>(gridDim.x) * EP_ROWS) {
        T* dst[EP_ROWS];
#pragma unroll
        for (int j = 0; j < EP_ROWS; ++j) {
            dst[j] = nullptr;
            if (p0 + j >= n_rows) continue;
            const int m = meta[p0 + j];
            if (m < 0) continue;  // pad row
            const int owner = m >> PEER_ROW_BITS;
            const int64_t row = m & PEER_ROW_MASK;
            if (owner >= world || row >= peer_rows_cap) {
                if (threadIdx.x == 0 && status) atomicOr(status, XMA_DEV_ID_OUT_OF_RANGE);
                continue;
            }
            dst[j] = static_cast<T*>(peer_rows[owner]) + row * width;
        }
        for (int64_t c = threadIdx.x; c < nvec; c += EP_ROW_THREADS) {
            Vec16<T> x[EP_ROWS];
#pragma unroll
            for (int j = 0; j < EP_ROWS; ++j)
                if (dst[j]) x[j] = load16_stream(rows + (p0 + j) * row_stride + c * V);
#pragma unroll
            for (int j = 0; j < EP_ROWS; ++j)
                if (dst[j]) store16(dst[j] + c * V, x[j]);
        }
    }
}

// Device words -> host memory that the device can address (pinned, mapped): a store instead of a
// copy-engine transfer, so a small read-back never queues behind bulk downloads.
__global__ void ep_publish_kernel(const int* __restrict__ src, int64_t n, int* __restrict__ host_words) {
    for (int64_t i = threadIdx.x; i < n; i += blockDim.x) host_words[i] = src[i];
    __threadfence_system();
}

static int ep_grid(int64_t rows) {
    int64_t want = ceil_div(rows, EP_ROWS);
    int64_t cap = static_cast<int64_t>(num_sms()) * 8;
    return static_cast<int>(want < 1 ? 1 : (want > cap ? cap : want));
}

template <typename T>
static int ep_dispatch_t(const void* src, int64_t src_stride, const int* sorted_expert, const int* sorted_scattered,
                         const void* coeff, int fan_out, const int* send_delta, int num_experts, int e_local,
                         int local_lo, int local_hi, int rank, int64_t rows, int64_t width, void* const* peer_rows,
                         int* const* peer_meta, int64_t peer_rows_cap, int* status, cudaStream_t stream) {
    if (width % Vec16<T>::N || src_stride % Vec16<T>::N || !is_aligned16(src)) return XMA_ERR_MISALIGNED;
    const int grid = ep_grid(rows);
    if (coeff)
        ep_dispatch_kernel<T, true><<<grid, EP_ROW_THREADS, 0, stream>>>(
            static_cast<const T*>(src), src_stride, sorted_expert, sorted_scattered, static_cast<const T*>(coeff),
            fan_out, send_delta, num_experts, e_local, local_lo, local_hi, rank, rows, width, peer_rows, peer_meta,
            peer_rows_cap, status);
    else
        ep_dispatch_kernel<T, false><<<grid, EP_ROW_THREADS, 0, stream>>>(
            static_cast<const T*>(src), src_stride, sorted_expert, sorted_scattered, nullptr, fan_out, send_delta,
            num_experts, e_local, local_lo, local_hi, rank, rows, width, peer_rows, peer_meta, peer_rows_cap, status);
    return static_cast<int>(cudaGetLastError());
}

template <typename T>
static int ep_copy_t(const void* rows, const int* meta, int64_t n_rows, int64_t width, void* out,
                     cudaStream_t stream) {
    if (width % Vec16<T>::N || !is_aligned16(rows) || !is_aligned16(out)) return XMA_ERR_MISALIGNED;
    const int grid = ep_grid(n_rows);
    if (rows == out)
        ep_copy_rows_kernel<T, true><<<grid, EP_ROW_THREADS, 0, stream>>>(static_cast<const T*>(rows), meta, n_rows,
                                                                          width, static_cast<T*>(out));
    else
        ep_copy_rows_kernel<T, false><<<grid, EP_ROW_THREADS, 0, stream>>>(static_cast<const T*>(rows), meta, n_rows,
                                                                           width, static_cast<T*>(out));
    return static_cast<int>(cudaGetLastError());
}

template <typename T>
static int ep_return_t(const void* rows, int64_t row_stride, const int* meta, int64_t n_rows, int64_t width,
                       int world, void* const* peer_rows, int64_t peer_rows_cap, int* status, cudaStream_t stream) {
    if (width % Vec16<T>::N || row_stride % Vec16<T>::N || !is_aligned16(rows)) return XMA_ERR_MISALIGNED;
    ep_return_kernel<T><<<ep_grid(n_rows), EP_ROW_THREADS, 0, stream>>>(
        static_cast<const T*>(rows), row_stride, meta, n_rows, width, world, peer_rows, peer_rows_cap, status);
    return static_cast<int>(cudaGetLastError());
}

}  // namespace xma

// ================================================================================================
// C ABI
// ================================================================================================
extern "C" {

int xma_b200_ep_plan(const int32_t* count_matrix, int world, int num_experts, int rank, int32_t* send_delta,
                     uint32_t* counts, int32_t* pad_offsets, int32_t* tile_prefix, int32_t* tile_expert,
                     int64_t tile_cap, int32_t* meta, int64_t meta_cap, int* device_status, cudaStream_t stream) {
    if (!count_matrix || !send_delta || !counts || !pad_offsets || !tile_prefix || !tile_expert || !meta)
        return XMA_ERR_NULL_POINTER;
    if (world <= 0 || world > xma::PEER_MAX_RANKS || rank < 0 || rank >= world || num_experts <= 0 ||
        num_experts > xma::EP_MAX_EXPERTS || num_experts % world || tile_cap < 0 || meta_cap < 0 ||
        tile_cap > 0x7fffffffLL / XMA_ROW_PAD)
        return XMA_ERR_BAD_SHAPE;
    xma::ep_plan_kernel<<<1, xma::EP_PLAN_THREADS, 0, stream>>>(count_matrix, world, num_experts, rank, send_delta,
                                                               counts, pad_offsets, tile_prefix, tile_expert,
                                                               static_cast<int>(tile_cap), meta, meta_cap,
                                                               device_status);
    return static_cast<int>(cudaGetLastError());
}

int xma_b200_ep_dispatch_part(const void* src, int dtype, int64_t src_row_stride, const int32_t* sorted_expert_idxs,
                              const int32_t* sorted_scattered_idxs, const void* coeff, int fan_out,
                              const int32_t* send_delta, int num_experts, int world, int rank, int local_lo,
                              int local_hi, int64_t rows, int64_t width, void* const* peer_rows,
                              int32_t* const* peer_meta, int64_t peer_rows_cap, int* device_status,
                              cudaStream_t stream) {
    if (rows == 0) return XMA_OK;
    if (!src || !sorted_expert_idxs || !sorted_scattered_idxs || !send_delta || !peer_rows)
        return XMA_ERR_NULL_POINTER;
    if (rows < 0 || width <= 0 || fan_out <= 0 || world <= 0 || world > xma::PEER_MAX_RANKS || rank < 0 ||
        rank >= world || num_experts <= 0 || num_experts % world || peer_rows_cap < 0)
        return XMA_ERR_BAD_SHAPE;
    if (rows > xma::PEER_ROW_MASK + 1LL) return XMA_ERR_TOO_LARGE;
    const int e_local = num_experts / world;
    if (local_lo < 0 || local_hi > e_local || local_lo > local_hi) return XMA_ERR_BAD_SHAPE;
    if (local_lo == local_hi) return XMA_OK;
#define XMA_EP_DISPATCH(T)                                                                                         \
    return xma::ep_dispatch_t<T>(src, src_row_stride, sorted_expert_idxs, sorted_scattered_idxs, coeff, fan_out,   \
                                 send_delta, num_experts, e_local, local_lo, local_hi, rank, rows, width,          \
                                 peer_rows, peer_meta, peer_rows_cap, device_status, stream)
    switch (dtype) {
        case XMA_F32: XMA_EP_DISPATCH(float);
        case XMA_F16: XMA_EP_DISPATCH(__half);
        case XMA_BF16: XMA_EP_DISPATCH(__nv_bfloat16);
    }
#undef XMA_EP_DISPATCH
    return XMA_ERR_BAD_DTYPE;
}

int xma_b200_ep_dispatch(const void* src, int dtype, int64_t src_row_stride, const int32_t* sorted_expert_idxs,
                         const int32_t* sorted_scattered_idxs, const void* coeff, int fan_out,
                         const int32_t* send_delta, int num_experts, int world, int rank, int64_t rows, int64_t width,
                         void* const* peer_rows, int32_t* const* peer_meta, int64_t peer_rows_cap,
                         int* device_status, cudaStream_t stream) {
    const int e_local = (world > 0 && num_experts > 0) ? num_experts / world : 0;
    return xma_b200_ep_dispatch_part(src, dtype, src_row_stride, sorted_expert_idxs, sorted_scattered_idxs, coeff,
                                     fan_out, send_delta, num_experts, world, rank, 0, e_local, rows, width, peer_rows,
                                     peer_meta, peer_rows_cap, device_status, stream);
}

int xma_b200_ep_copy_rows(const void* rows, int dtype, const int32_t* meta, int64_t n_rows, int64_t width, void* out,
                          cudaStream_t stream) {
    if (n_rows == 0) return XMA_OK;
    if (!rows || !meta || !out) return XMA_ERR_NULL_POINTER;
    if (n_rows < 0 || width <= 0) return XMA_ERR_BAD_SHAPE;
    switch (dtype) {
        case XMA_F32: return xma::ep_copy_t<float>(rows, meta, n_rows, width, out, stream);
        case XMA_F16: return xma::ep_copy_t<__half>(rows, meta, n_rows, width, out, stream);
        case XMA_BF16: return xma::ep_copy_t<__nv_bfloat16>(rows, meta, n_rows, width, out, stream);
    }
    return XMA_ERR_BAD_DTYPE;
}

int xma_b200_ep_publish(const int32_t* src, int64_t n, int32_t* host_words, cudaStream_t stream) {
    if (n == 0) return XMA_OK;
    if (!src || !host_words) return XMA_ERR_NULL_POINTER;
    if (n < 0) return XMA_ERR_BAD_SHAPE;
    xma::ep_publish_kernel<<<1, 256, 0, stream>>>(src, n, host_words);
    return static_cast<int>(cudaGetLastError());
}

int xma_b200_ep_return(const void* rows, int dtype, int64_t row_stride, const int32_t* meta, int64_t n_rows,
                       int64_t width, int world, void* const* peer_rows, int64_t peer_rows_cap, int* device_status,
                       cudaStream_t stream) {
    if (n_rows == 0) return XMA_OK;
    if (!rows || !meta || !peer_rows) return XMA_ERR_NULL_POINTER;
    if (n_rows < 0 || width <= 0 || world <= 0 || world > xma::PEER_MAX_RANKS || peer_rows_cap < 0)
        return XMA_ERR_BAD_SHAPE;
    switch (dtype) {
        case XMA_F32:
            return xma::ep_return_t<float>(rows, row_stride, meta, n_rows, width, world, peer_rows, peer_rows_cap,
                                           device_status, stream);
        case XMA_F16:
            return xma::ep_return_t<__half>(rows, row_stride, meta, n_rows, width, world, peer_rows, peer_rows_cap,
                                            device_status, stream);
        case XMA_BF16:
            return xma::ep_return_t<__nv_bfloat16>(rows, row_stride, meta, n_rows, width, world, peer_rows,
                                                   peer_rows_cap, device_status, stream);
    }
    return XMA_ERR_BAD_DTYPE;
}

// ---- exchange buffers: device memory that other processes of the node map ------------------------
// Plain cudaMalloc memory (zero-filled) so that it can be exported with the CUDA IPC calls.
int xma_b200_exchange_alloc(int64_t bytes, void** out_ptr) {
    if (!out_ptr) return XMA_ERR_NULL_POINTER;
    if (bytes <= 0) return XMA_ERR_BAD_SHAPE;
    void* p = nullptr;
    XMA_CUDA_TRY(cudaMalloc(&p, static_cast<size_t>(bytes)));
    cudaError_t e = cudaMemset(p, 0, static_cast<size_t>(bytes));
    if (e != cudaSuccess) {
        cudaFree(p);
        return static_cast<int>(e);
    }
    *out_ptr = p;
    return XMA_OK;
}

int xma_b200_exchange_free(void* ptr) {
    if (!ptr) return XMA_OK;
    return static_cast<int>(cudaFree(ptr));
}

int xma_b200_exchange_handle_bytes(void) { return static_cast<int>(sizeof(cudaIpcMemHandle_t)); }

// handle_out: xma_b200_exchange_handle_bytes() bytes that another process passes to _open.
int xma_b200_exchange_export(void* ptr, void* handle_out) {
    if (!ptr || !handle_out) return XMA_ERR_NULL_POINTER;
    cudaIpcMemHandle_t h;
    XMA_CUDA_TRY(cudaIpcGetMemHandle(&h, ptr));
    memcpy(handle_out, &h, sizeof(h));
    return XMA_OK;
}

// Maps another process's exchange buffer into this process for the current device (peer access
// between the two devices is enabled by the driver on first use).
int xma_b200_exchange_open(const void* handle, void** out_ptr) {
    if (!handle || !out_ptr) return XMA_ERR_NULL_POINTER;
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, sizeof(h));
    void* p = nullptr;
    XMA_CUDA_TRY(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
    *out_ptr = p;
    return XMA_OK;
}

int xma_b200_exchange_close(void* ptr) {
    if (!ptr) return XMA_OK;
    return static_cast<int>(cudaIpcCloseMemHandle(ptr));
}

}  // extern "C"
