// Row movement kernels of the MoE hot path (pure HBM-bandwidth work, 128-bit accesses):
//   * gather_rows   : token rows -> expert-sorted (padded) rows, optional per-row coefficient.
//                     Replaces `group` (xma/layers/moe/triton_implementation/group_kernel.py:69-100).
//   * combine_rows  : y[t] = sum_k w[t,k] * Ys[t*K+k]  (fp32 accumulate, one rounding). Replaces the
//                     `bmm` combine of xma/layers/moe/triton_implementation/__init__.py:100-101 and
//                     the `.view(T,K,H).sum(-2)` of :70.
//   * combine_bwd   : d_router_weights[t,k] = <Ys[t*K+k], dY[t]> (same file, :130-131).
//   * spread_rows   : the token-major form of gather_rows: a token's row is read once and written to the K
//                     grouped rows of its slots (gather_rows reads it K times); optionally fused with
//                     combine_bwd, which reads the same dY row.
#include "common.cuh"

namespace xma {

constexpr int ROW_THREADS = 256;

// out[p, :] = src[row_src[p] / fan_out, :] * coeff[row_src[p]]   (zeros where row_src[p] < 0)
// A CTA moves GATHER_ROWS rows per iteration so that every thread has that many independent
// 128-bit loads in flight (one row alone does not cover the HBM latency-bandwidth product).
constexpr int GATHER_ROWS = 4;

template <typename T, bool HAS_COEFF>
__global__ void __launch_bounds__(ROW_THREADS)
gather_rows_kernel(const T* __restrict__ src, int64_t src_stride, const int* __restrict__ row_src,
                   const T* __restrict__ coeff, int fan_out, int64_t rows, const int* __restrict__ rows_in_use,
                   int64_t width, T* __restrict__ out, int64_t out_stride) {
    constexpr int V = Vec16<T>::N;
    const int64_t limit = rows_in_use ? min(rows, static_cast<int64_t>(*rows_in_use)) : rows;
    const int64_t nvec = width / V;
    for (int64_t p0 = static_cast<int64_t>(blockIdx.x) * GATHER_ROWS; p0 < limit;
         p0 += static_cast<int64_t>(gridDim.x) * GATHER_ROWS) {
        int f[GATHER_ROWS];
        float cf[GATHER_ROWS];
#pragma unroll
        for (int j = 0; j < GATHER_ROWS; ++j) {
            f[j] = (p0 + j < limit) ? row_src[p0 + j] : -2;  // -2: row does not exist, -1: pad row
            cf[j] = 1.0f;
            if (HAS_COEFF && f[j] >= 0) cf[j] = to_f32(coeff[f[j]]);
        }
        for (int64_t c = threadIdx.x; c < nvec; c += ROW_THREADS) {
            Vec16<T> x[GATHER_ROWS];
#pragma unroll
            for (int j = 0; j < GATHER_ROWS; ++j) {
                if (f[j] >= 0) {
                    x[j] = load16(src + static_cast<int64_t>(f[j] / fan_out) * src_stride + c * V);
                } else {
#pragma unroll
                    for (int i = 0; i < V; ++i) x[j].v[i] = from_f32<T>(0.0f);
                }
            }
#pragma unroll
            for (int j = 0; j < GATHER_ROWS; ++j) {
                if (f[j] == -2) continue;
                if (HAS_COEFF && f[j] >= 0) {
#pragma unroll
                    for (int i = 0; i < V; ++i) x[j].v[i] = from_f32<T>(to_f32(x[j].v[i]) * cf[j]);
                }
                store16_stream(out + (p0 + j) * out_stride + c * V, x[j]);
            }
        }
    }
}

// y[t, :] = sum_k w[t,k] * ys[row(t*K + k), :]; w == nullptr means plain sum; row(f) = row_index[f]
// when an index is given (rows kept in another order), f otherwise.
template <typename T, bool HAS_W>
__global__ void __launch_bounds__(ROW_THREADS)
combine_rows_kernel(const T* __restrict__ ys, int64_t ys_stride, const T* __restrict__ w,
                    const int* __restrict__ row_index, int K, int64_t tokens, int64_t width, T* __restrict__ y,
                    int64_t y_stride) {
    constexpr int V = Vec16<T>::N;
    const int64_t nvec = width / V;
    for (int64_t t = blockIdx.x; t < tokens; t += gridDim.x) {
        for (int64_t c = threadIdx.x; c < nvec; c += ROW_THREADS) {
            float acc[V];
#pragma unroll
            for (int j = 0; j < V; ++j) acc[j] = 0.0f;
            for (int k = 0; k < K; ++k) {
                const float wk = HAS_W ? to_f32(w[t * K + k]) : 1.0f;
                const int64_t r = row_index ? row_index[t * K + k] : t * K + k;
                Vec16<T> x = load16_stream(ys + r * ys_stride + c * V);
#pragma unroll
                for (int j = 0; j < V; ++j) acc[j] = fmaf(wk, to_f32(x.v[j]), acc[j]);
            }
            Vec16<T> o;
#pragma unroll
            for (int j = 0; j < V; ++j) o.v[j] = from_f32<T>(acc[j]);
            store16(y + t * y_stride + c * V, o);
        }
    }
}

// dw[t, k] = sum_h ys[row(t*K+k), h] * dy[t, h]
// Each warp owns whole (token, slot) rows, so a dot product is one warp reduction and the CTA never
// synchronises (dy[t] is re-read from L1/L2 by the warps that share a token).
template <typename T>
__global__ void __launch_bounds__(ROW_THREADS)
combine_bwd_kernel(const T* __restrict__ ys, int64_t ys_stride, const T* __restrict__ dy, int64_t dy_stride,
                   const int* __restrict__ row_index, int K, int64_t tokens, int64_t width, T* __restrict__ dw) {
    constexpr int V = Vec16<T>::N;
    constexpr int WARPS = ROW_THREADS / 32;
    const int64_t nvec = width / V;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int64_t pairs = tokens * K;
    for (int64_t q = static_cast<int64_t>(blockIdx.x) * WARPS + warp; q < pairs;
         q += static_cast<int64_t>(gridDim.x) * WARPS) {
        {
            const int64_t t = q / K;
            const T* dy_row = dy + t * dy_stride;
            const int64_t r = row_index ? row_index[q] : q;
            const T* ys_row = ys + r * ys_stride;
            float acc = 0.0f;
            int64_t c = lane;
            for (; c + 32 < nvec; c += 64) {  // two packets of each operand in flight
                Vec16<T> a0 = load16_stream(ys_row + c * V), a1 = load16_stream(ys_row + (c + 32) * V);
                Vec16<T> b0 = load16(dy_row + c * V), b1 = load16(dy_row + (c + 32) * V);
#pragma unroll
                for (int j = 0; j < V; ++j) acc = fmaf(to_f32(a0.v[j]), to_f32(b0.v[j]), acc);
#pragma unroll
                for (int j = 0; j < V; ++j) acc = fmaf(to_f32(a1.v[j]), to_f32(b1.v[j]), acc);
            }
            for (; c < nvec; c += 32) {
                Vec16<T> a0 = load16_stream(ys_row + c * V);
                Vec16<T> b0 = load16(dy_row + c * V);
#pragma unroll
                for (int j = 0; j < V; ++j) acc = fmaf(to_f32(a0.v[j]), to_f32(b0.v[j]), acc);
            }
#pragma unroll
            for (int o = 16; o >= 1; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
            if (lane == 0) dw[q] = from_f32<T>(acc);
        }
    }
}

// Token-major scatter: for every token t and slot k < K
//   out[row_dst[t*K + k], :] = src[t, :] * coeff[t*K + k]                 (coeff == nullptr: 1)
//   dw[t*K + k]              = <ys[t*K + k, :], src[t, :]>                (HAS_DOT; fp32 accumulate)
// followed by the zero fill of every expert's pad rows [pad_offsets[e] + counts[e], pad_offsets[e+1]).
// One CTA per token: a thread keeps its packets of the token's row in registers, so the row is read once
// (gather_rows fetches it once per slot, and the backward's combine_bwd reads it again); with top-8 routing
// that is 2.1 instead of 3.1 passes over [rows, width] for the backward pair and 1.1 instead of 2 forward.
constexpr int SPREAD_K = 8;  // slots handled per pass over the registers (dot accumulators held per thread)

template <typename T, bool HAS_COEFF, bool HAS_DOT>
__global__ void __launch_bounds__(ROW_THREADS)
spread_rows_kernel(const T* __restrict__ src, int64_t src_stride, const int* __restrict__ row_dst,
                   const T* __restrict__ coeff, const T* __restrict__ ys, int64_t ys_stride, T* __restrict__ dw,
                   int K, int64_t tokens, int64_t width, T* __restrict__ out, int64_t out_stride,
                   const unsigned* __restrict__ counts, const int* __restrict__ pad_offsets, int E) {
    constexpr int V = Vec16<T>::N;
    constexpr int WARPS = ROW_THREADS / 32;
    __shared__ float s_part[WARPS][SPREAD_K];
    __shared__ int s_dst[32];
    __shared__ float s_cf[32];
    const int64_t nvec = width / V;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int64_t t = blockIdx.x; t < tokens; t += gridDim.x) {
        __syncthreads();  // s_dst / s_cf / s_part of the previous token are no longer read
        if (threadIdx.x < K) {
            s_dst[threadIdx.x] = row_dst[t * K + threadIdx.x];
            s_cf[threadIdx.x] = HAS_COEFF ? to_f32(coeff[t * K + threadIdx.x]) : 1.0f;
        }
        __syncthreads();
        const T* src_row = src + t * src_stride;
        for (int k0 = 0; k0 < K; k0 += SPREAD_K) {
            float acc[SPREAD_K];
#pragma unroll
            for (int j = 0; j < SPREAD_K; ++j) acc[j] = 0.0f;
            for (int64_t c = threadIdx.x; c < nvec; c += ROW_THREADS) {
                const Vec16<T> x = load16(src_row + c * V);
                float xf[V];
#pragma unroll
                for (int i = 0; i < V; ++i) xf[i] = to_f32(x.v[i]);
                Vec16<T> y[SPREAD_K];
                if (HAS_DOT) {
#pragma unroll
                    for (int j = 0; j < SPREAD_K; ++j)
                        if (k0 + j < K) y[j] = load16_stream(ys + (t * K + k0 + j) * ys_stride + c * V);
                }
#pragma unroll
                for (int j = 0; j < SPREAD_K; ++j) {
                    if (k0 + j >= K) break;
                    if (HAS_DOT) {
#pragma unroll
                        for (int i = 0; i < V; ++i) acc[j] = fmaf(to_f32(y[j].v[i]), xf[i], acc[j]);
                    }
                    const int dst = s_dst[k0 + j];
                    if (dst < 0) continue;
                    Vec16<T> o = x;
                    if (HAS_COEFF) {
                        const float cf = s_cf[k0 + j];
#pragma unroll
                        for (int i = 0; i < V; ++i) o.v[i] = from_f32<T>(xf[i] * cf);
                    }
                    store16_stream(out + static_cast<int64_t>(dst) * out_stride + c * V, o);
                }
            }
            if (HAS_DOT) {
#pragma unroll
                for (int j = 0; j < SPREAD_K; ++j) {
#pragma unroll
                    for (int o = 16; o >= 1; o >>= 1) acc[j] += __shfl_xor_sync(0xffffffffu, acc[j], o);
                }
                if (k0 > 0) __syncthreads();  // the previous pass's partial sums have been read
                if (lane == 0) {
#pragma unroll
                    for (int j = 0; j < SPREAD_K; ++j) s_part[warp][j] = acc[j];
                }
                __syncthreads();
                if (threadIdx.x < SPREAD_K && k0 + threadIdx.x < K) {
                    float sum = 0.0f;
#pragma unroll
                    for (int w = 0; w < WARPS; ++w) sum += s_part[w][threadIdx.x];
                    dw[t * K + k0 + threadIdx.x] = from_f32<T>(sum);
                }
            }
        }
    }
    // pad rows of the grouped layout (at most 127 per expert)
    const int64_t candidates = static_cast<int64_t>(E) * XMA_ROW_PAD;
    for (int64_t i = blockIdx.x; i < candidates; i += gridDim.x) {
        const int e = static_cast<int>(i / XMA_ROW_PAD);
        const int64_t p = static_cast<int64_t>(pad_offsets[e]) + counts[e] + (i % XMA_ROW_PAD);
        if (p >= pad_offsets[e + 1]) continue;  // uniform for the CTA
        Vec16<T> z;
#pragma unroll
        for (int j = 0; j < V; ++j) z.v[j] = from_f32<T>(0.0f);
        for (int64_t c = threadIdx.x; c < nvec; c += ROW_THREADS) store16(out + p * out_stride + c * V, z);
    }
}

static int row_grid(int64_t rows, int rows_per_cta = 1) {
    int64_t want = ceil_div(rows, rows_per_cta);
    int64_t cap = static_cast<int64_t>(num_sms()) * 8;
    return static_cast<int>(want < 1 ? 1 : (want > cap ? cap : want));
}

template <typename T>
static int gather_impl(const void* src, int64_t src_stride, const int* row_src, const void* coeff, int fan_out,
                       int64_t rows, const int* rows_in_use, int64_t width, void* out, int64_t out_stride,
                       cudaStream_t stream) {
    constexpr int V = Vec16<T>::N;
    if (width % V || src_stride % V || out_stride % V || !is_aligned16(src) || !is_aligned16(out))
        return XMA_ERR_MISALIGNED;
    const int grid = row_grid(rows, GATHER_ROWS);
    if (coeff)
        gather_rows_kernel<T, true><<<grid, ROW_THREADS, 0, stream>>>(
            static_cast<const T*>(src), src_stride, row_src, static_cast<const T*>(coeff), fan_out, rows,
            rows_in_use, width, static_cast<T*>(out), out_stride);
    else
        gather_rows_kernel<T, false><<<grid, ROW_THREADS, 0, stream>>>(
            static_cast<const T*>(src), src_stride, row_src, nullptr, fan_out, rows, rows_in_use, width,
            static_cast<T*>(out), out_stride);
    return static_cast<int>(cudaGetLastError());
}

template <typename T>
static int combine_impl(const void* ys, int64_t ys_stride, const void* w, const int* row_index, int K,
                        int64_t tokens, int64_t width, void* y, int64_t y_stride, cudaStream_t stream) {
    constexpr int V = Vec16<T>::N;
    if (width % V || ys_stride % V || y_stride % V || !is_aligned16(ys) || !is_aligned16(y))
        return XMA_ERR_MISALIGNED;
    const int grid = row_grid(tokens);
    if (w)
        combine_rows_kernel<T, true><<<grid, ROW_THREADS, 0, stream>>>(
            static_cast<const T*>(ys), ys_stride, static_cast<const T*>(w), row_index, K, tokens, width,
            static_cast<T*>(y), y_stride);
    else
        combine_rows_kernel<T, false><<<grid, ROW_THREADS, 0, stream>>>(
            static_cast<const T*>(ys), ys_stride, nullptr, row_index, K, tokens, width, static_cast<T*>(y), y_stride);
    return static_cast<int>(cudaGetLastError());
}

template <typename T>
static int combine_bwd_impl(const void* ys, int64_t ys_stride, const void* dy, int64_t dy_stride,
                            const int* row_index, int K, int64_t tokens, int64_t width, void* dw,
                            cudaStream_t stream) {
    constexpr int V = Vec16<T>::N;
    if (width % V || ys_stride % V || dy_stride % V || !is_aligned16(ys) || !is_aligned16(dy))
        return XMA_ERR_MISALIGNED;
    combine_bwd_kernel<T><<<row_grid(tokens * K, ROW_THREADS / 32), ROW_THREADS, 0, stream>>>(
        static_cast<const T*>(ys), ys_stride, static_cast<const T*>(dy), dy_stride, row_index, K, tokens, width,
        static_cast<T*>(dw));
    return static_cast<int>(cudaGetLastError());
}

template <typename T>
static int spread_impl(const void* src, int64_t src_stride, const int* row_dst, const void* coeff, const void* ys,
                       int64_t ys_stride, void* dw, int K, int64_t tokens, int64_t width, void* out,
                       int64_t out_stride, const unsigned* counts, const int* pad_offsets, int E, cudaStream_t stream) {
    constexpr int V = Vec16<T>::N;
    if (width % V || src_stride % V || out_stride % V || !is_aligned16(src) || !is_aligned16(out))
        return XMA_ERR_MISALIGNED;
    if (ys && (ys_stride % V || !is_aligned16(ys))) return XMA_ERR_MISALIGNED;
    const int64_t work = tokens > static_cast<int64_t>(E) * XMA_ROW_PAD ? tokens : static_cast<int64_t>(E) * XMA_ROW_PAD;
    const int grid = row_grid(work);
#define XMA_SPREAD(COEFF, DOT)                                                                               \
    spread_rows_kernel<T, COEFF, DOT><<<grid, ROW_THREADS, 0, stream>>>(                                     \
        static_cast<const T*>(src), src_stride, row_dst, static_cast<const T*>(coeff), static_cast<const T*>(ys), \
        ys_stride, static_cast<T*>(dw), K, tokens, width, static_cast<T*>(out), out_stride, counts, pad_offsets, E)
    if (coeff && ys) XMA_SPREAD(true, true);
    else if (coeff) XMA_SPREAD(true, false);
    else if (ys) XMA_SPREAD(false, true);
    else XMA_SPREAD(false, false);
#undef XMA_SPREAD
    return static_cast<int>(cudaGetLastError());
}

}  // namespace xma

extern "C" {

int xma_b200_gather_rows(const void* src, int dtype, int64_t src_row_stride, const int32_t* row_src,
                         const void* coeff, int fan_out, int64_t rows, const int32_t* rows_in_use, int64_t width,
                         void* out, int64_t out_row_stride, cudaStream_t stream) {
    if (rows > 0 && (!src || !row_src || !out)) return XMA_ERR_NULL_POINTER;
    if (rows < 0 || width <= 0 || fan_out <= 0) return XMA_ERR_BAD_SHAPE;
    if (rows == 0) return XMA_OK;
    switch (dtype) {
        case XMA_F32:
            return xma::gather_impl<float>(src, src_row_stride, row_src, coeff, fan_out, rows, rows_in_use, width,
                                           out, out_row_stride, stream);
        case XMA_F16:
            return xma::gather_impl<__half>(src, src_row_stride, row_src, coeff, fan_out, rows, rows_in_use, width,
                                            out, out_row_stride, stream);
        case XMA_BF16:
            return xma::gather_impl<__nv_bfloat16>(src, src_row_stride, row_src, coeff, fan_out, rows, rows_in_use,
                                                   width, out, out_row_stride, stream);
    }
    return XMA_ERR_BAD_DTYPE;
}

int xma_b200_combine_rows(const void* ys, int dtype, int64_t ys_row_stride, const void* weights,
                          const int32_t* row_index, int top_k, int64_t tokens, int64_t width, void* y,
                          int64_t y_row_stride, cudaStream_t stream) {
    if (tokens > 0 && (!ys || !y)) return XMA_ERR_NULL_POINTER;
    if (tokens < 0 || width <= 0 || top_k <= 0) return XMA_ERR_BAD_SHAPE;
    if (tokens == 0) return XMA_OK;
    switch (dtype) {
        case XMA_F32:
            return xma::combine_impl<float>(ys, ys_row_stride, weights, row_index, top_k, tokens, width, y,
                                            y_row_stride, stream);
        case XMA_F16:
            return xma::combine_impl<__half>(ys, ys_row_stride, weights, row_index, top_k, tokens, width, y,
                                             y_row_stride, stream);
        case XMA_BF16:
            return xma::combine_impl<__nv_bfloat16>(ys, ys_row_stride, weights, row_index, top_k, tokens, width, y,
                                                    y_row_stride, stream);
    }
    return XMA_ERR_BAD_DTYPE;
}

int xma_b200_combine_bwd(const void* ys, int dtype, int64_t ys_row_stride, const void* dy, int64_t dy_row_stride,
                         const int32_t* row_index, int top_k, int64_t tokens, int64_t width, void* d_weights,
                         cudaStream_t stream) {
    if (tokens > 0 && (!ys || !dy || !d_weights)) return XMA_ERR_NULL_POINTER;
    if (tokens < 0 || width <= 0 || top_k <= 0) return XMA_ERR_BAD_SHAPE;
    if (tokens == 0) return XMA_OK;
    switch (dtype) {
        case XMA_F32:
            return xma::combine_bwd_impl<float>(ys, ys_row_stride, dy, dy_row_stride, row_index, top_k, tokens,
                                                width, d_weights, stream);
        case XMA_F16:
            return xma::combine_bwd_impl<__half>(ys, ys_row_stride, dy, dy_row_stride, row_index, top_k, tokens,
                                                 width, d_weights, stream);
        case XMA_BF16:
            return xma::combine_bwd_impl<__nv_bfloat16>(ys, ys_row_stride, dy, dy_row_stride, row_index, top_k,
                                                        tokens, width, d_weights, stream);
    }
    return XMA_ERR_BAD_DTYPE;
}

int xma_b200_spread_rows(const void* src, int dtype, int64_t src_row_stride, const int32_t* row_dst, const void* coeff,
                         const void* ys, int64_t ys_row_stride, void* d_weights, int top_k, int64_t tokens,
                         int64_t width, void* out, int64_t out_row_stride, const uint32_t* counts,
                         const int32_t* pad_offsets, int num_experts, cudaStream_t stream) {
    if (!row_dst || !out || !counts || !pad_offsets || (tokens > 0 && !src)) return XMA_ERR_NULL_POINTER;
    if ((ys == nullptr) != (d_weights == nullptr)) return XMA_ERR_NULL_POINTER;
    if (tokens < 0 || width <= 0 || top_k <= 0 || top_k > 32 || num_experts <= 0) return XMA_ERR_BAD_SHAPE;
    switch (dtype) {
        case XMA_F32:
            return xma::spread_impl<float>(src, src_row_stride, row_dst, coeff, ys, ys_row_stride, d_weights, top_k,
                                           tokens, width, out, out_row_stride, counts, pad_offsets, num_experts,
                                           stream);
        case XMA_F16:
            return xma::spread_impl<__half>(src, src_row_stride, row_dst, coeff, ys, ys_row_stride, d_weights, top_k,
                                            tokens, width, out, out_row_stride, counts, pad_offsets, num_experts,
                                            stream);
        case XMA_BF16:
            return xma::spread_impl<__nv_bfloat16>(src, src_row_stride, row_dst, coeff, ys, ys_row_stride, d_weights,
                                                   top_k, tokens, width, out, out_row_stride, counts, pad_offsets,
                                                   num_experts, stream);
    }
    return XMA_ERR_BAD_DTYPE;
}

}  // extern "C"
