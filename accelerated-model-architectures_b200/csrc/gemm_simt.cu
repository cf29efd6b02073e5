// CUDA-core grouped GEMMs for the MoE experts: any dtype (fp32 math for fp32 inputs), any shape.
// They serve the shapes and dtypes the tensor-core path does not take (fp32, widths that are not
// multiples of 8) and are the on-device cross-check for it. Semantics follow scatter2scatter
// (xma/layers/moe/triton_implementation/scatter_kernel.py:137-183) and group_bwd_W
// (xma/layers/moe/triton_implementation/group_backward_kernel.py:102-128) on the padded grouped
// row layout produced by count_sort.
#include "gemm_internal.h"

namespace xma {

constexpr int ST_BM = 64, ST_BN = 64, ST_BK = 16, ST_THREADS = 256;

// acc[4][4] += A(m0 + .., k) * B(k, n0 + ..) over k in [0, k_len). A(m,k) = a[m*a_ms + k*a_ks],
// B(k,n) = b[k*b_ks + n*b_ns]; rows >= m_lim / columns >= n_lim read as zero.
template <typename T>
__device__ __forceinline__ void simt_tile(const T* __restrict__ a, int64_t a_ms, int64_t a_ks, int64_t m_lim,
                                          const T* __restrict__ b, int64_t b_ks, int64_t b_ns, int64_t n_lim,
                                          int64_t k_len, float (&acc)[4][4]) {
    __shared__ float sa[ST_BK][ST_BM + 4];
    __shared__ float sb[ST_BK][ST_BN + 4];
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;  // 16 x 16 threads, 4 x 4 outputs each
    const bool a_kfast = (a_ks == 1), b_kfast = (b_ks == 1);

    for (int64_t k0 = 0; k0 < k_len; k0 += ST_BK) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            int m, k;
            if (a_kfast) {
                m = tid >> 2;
                k = (tid & 3) * 4 + j;
            } else {
                m = tid & 63;
                k = (tid >> 6) + 4 * j;
            }
            float v = 0.0f;
            if (m < m_lim && k0 + k < k_len) v = to_f32(a[m * a_ms + (k0 + k) * a_ks]);
            sa[k][m] = v;
            int n, kb;
            if (b_kfast) {
                n = tid >> 2;
                kb = (tid & 3) * 4 + j;
            } else {
                n = tid & 63;
                kb = (tid >> 6) + 4 * j;
            }
            float w = 0.0f;
            if (n < n_lim && k0 + kb < k_len) w = to_f32(b[(k0 + kb) * b_ks + n * b_ns]);
            sb[kb][n] = w;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < ST_BK; ++k) {
            float av[4], bv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) av[i] = sa[k][ty * 4 + i];
#pragma unroll
            for (int i = 0; i < 4; ++i) bv[i] = sb[k][tx * 4 + i];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
        }
        __syncthreads();
    }
}

// grid = (2 * tile_cap, ceil(N / 64)): two 64-row CTAs per 128-row padded tile.
template <typename T>
__global__ void __launch_bounds__(ST_THREADS)
rows_gemm_simt_kernel(const T* __restrict__ a, int64_t a_stride, const T* __restrict__ w, int w_layout,
                      T* __restrict__ out, int64_t out_stride, const int* __restrict__ row_map,
                      void* const* __restrict__ out_peers, int peer_world, int64_t peer_rows_cap,
                      const int* __restrict__ tile_expert, const int* __restrict__ tile_prefix, int E, int64_t kd,
                      int64_t n, int* __restrict__ status) {
    const int tile = blockIdx.x >> 1;
    if (tile >= tile_prefix[E]) return;
    const int e = tile_expert[tile];
    if (e < 0 || e >= E) return;
    const int64_t r0 = static_cast<int64_t>(blockIdx.x) * ST_BM;
    const int64_t n0 = static_cast<int64_t>(blockIdx.y) * ST_BN;
    const T* we = w + static_cast<int64_t>(e) * kd * n;
    float acc[4][4] = {};
    if (w_layout == W_NK)
        simt_tile<T>(a + r0 * a_stride, a_stride, 1, ST_BM, we + n0 * kd, 1, kd, n - n0, kd, acc);
    else
        simt_tile<T>(a + r0 * a_stride, a_stride, 1, ST_BM, we + n0, n, 1, n - n0, kd, acc);
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int64_t r = r0 + ty * 4 + i;
        int64_t dst = r;
        if (row_map) dst = row_map[r];
        if (dst < 0) continue;
        T* base = out;
        if (out_peers) {  // (rank << 24) | row of that rank's buffer; words outside the table are skipped and flagged
            const int64_t owner = dst >> PEER_ROW_BITS;
            dst &= PEER_ROW_MASK;
            if (owner >= peer_world || dst >= peer_rows_cap) {
                if (status && tx == 0) atomicOr(status, XMA_DEV_ID_OUT_OF_RANGE);
                continue;
            }
            base = static_cast<T*>(out_peers[owner]);
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int64_t c = n0 + tx * 4 + j;
            if (c < n) base[dst * out_stride + c] = from_f32<T>(acc[i][j]);
        }
    }
}

// grid = (ceil(M/64), ceil(N/64), E). Experts without rows get an all-zero dW tile.
template <typename T>
__global__ void __launch_bounds__(ST_THREADS)
dw_gemm_simt_kernel(const T* __restrict__ x, int64_t x_stride, const T* __restrict__ y, int64_t y_stride,
                    const uint32_t* __restrict__ counts, const int* __restrict__ pad_offsets, int64_t m, int64_t n,
                    T* __restrict__ dw) {
    const int e = blockIdx.z;
    const int64_t m0 = static_cast<int64_t>(blockIdx.x) * ST_BM;
    const int64_t n0 = static_cast<int64_t>(blockIdx.y) * ST_BN;
    const int64_t r0 = pad_offsets[e];
    const int64_t rows = counts[e];
    float acc[4][4] = {};
    simt_tile<T>(x + r0 * x_stride + m0, 1, x_stride, m - m0, y + r0 * y_stride + n0, y_stride, 1, n - n0, rows, acc);
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    T* dst = dw + static_cast<int64_t>(e) * m * n;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int64_t r = m0 + ty * 4 + i;
        if (r >= m) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int64_t c = n0 + tx * 4 + j;
            if (c < n) dst[r * n + c] = from_f32<T>(acc[i][j]);
        }
    }
}

template <typename T>
static int rows_gemm_simt_t(const RowsGemmArgs& g) {
    const int64_t i_width = (g.epilogue == EPI_SWIGLU) ? g.n / 2 : g.n;
    // Where the raw contraction lands: the gate|up buffer for the SwiGLU forward, the first half of
    // the output for its backward (rewritten in place afterwards), the output otherwise.
    T* raw = static_cast<T*>(g.epilogue == EPI_SWIGLU ? g.aux : g.out);
    const int64_t raw_stride = (g.epilogue == EPI_SWIGLU) ? g.aux_stride : g.out_stride;
    const bool plain = (g.epilogue == EPI_PLAIN || g.epilogue == EPI_PLAIN_PEER);
    const int* row_map = plain ? g.row_map : nullptr;
    void* const* out_peers = (g.epilogue == EPI_PLAIN_PEER) ? g.out_peers : nullptr;
    dim3 grid(static_cast<unsigned>(2 * g.tile_cap), static_cast<unsigned>(ceil_div(g.n, ST_BN)));
    if (grid.y > 65535) return XMA_ERR_TOO_LARGE;
    rows_gemm_simt_kernel<T><<<grid, ST_THREADS, 0, g.stream>>>(
        static_cast<const T*>(g.a), g.a_stride, static_cast<const T*>(g.w), g.w_layout, raw, raw_stride, row_map,
        out_peers, g.peer_world, g.peer_rows_cap, g.tile_expert, g.tile_prefix, g.num_experts, g.kd, g.n,
        g.device_status);
    XMA_CUDA_TRY(cudaGetLastError());
    const int64_t rows = g.tile_cap * XMA_ROW_PAD;
    if (g.epilogue == EPI_SWIGLU) {
        const T* gu = static_cast<const T*>(g.aux);
        return swiglu_fwd_launch(gu, g.aux_stride, gu + i_width, g.aux_stride, g.out, g.out_stride, g.dtype, rows,
                                 i_width, g.stream);
    }
    if (g.epilogue == EPI_DSWIGLU) {
        const T* gu = static_cast<const T*>(g.aux);
        T* o = static_cast<T*>(g.out);
        return swiglu_bwd_launch(gu, g.aux_stride, gu + i_width, g.aux_stride, o, g.out_stride, o, g.out_stride,
                                 o + i_width, g.out_stride, g.dtype, rows, i_width, g.stream);
    }
    return XMA_OK;
}

template <typename T>
static int dw_gemm_simt_t(const DwGemmArgs& g) {
    dim3 grid(static_cast<unsigned>(ceil_div(g.m, ST_BM)), static_cast<unsigned>(ceil_div(g.n, ST_BN)),
              static_cast<unsigned>(g.num_experts));
    if (grid.y > 65535 || grid.z > 65535) return XMA_ERR_TOO_LARGE;
    dw_gemm_simt_kernel<T><<<grid, ST_THREADS, 0, g.stream>>>(static_cast<const T*>(g.x), g.x_stride,
                                                              static_cast<const T*>(g.y), g.y_stride, g.counts,
                                                              g.pad_offsets, g.m, g.n, static_cast<T*>(g.dw));
    return static_cast<int>(cudaGetLastError());
}

int rows_gemm_simt(const RowsGemmArgs& g) {
    // the interleaved SwiGLU epilogues exist on the tensor-core kernels only (the caller composes
    // a plain GEMM with the stand-alone swiglu_packed kernels instead)
    if (g.epilogue == EPI_SWIGLU_PACKED || g.epilogue == EPI_DSWIGLU_PACKED) return XMA_ERR_UNSUPPORTED;
    if (g.tile_cap == 0) return XMA_OK;
    switch (g.dtype) {
        case XMA_F32: return rows_gemm_simt_t<float>(g);
        case XMA_F16: return rows_gemm_simt_t<__half>(g);
        case XMA_BF16: return rows_gemm_simt_t<__nv_bfloat16>(g);
    }
    return XMA_ERR_BAD_DTYPE;
}

int dw_gemm_simt(const DwGemmArgs& g) {
    switch (g.dtype) {
        case XMA_F32: return dw_gemm_simt_t<float>(g);
        case XMA_F16: return dw_gemm_simt_t<__half>(g);
        case XMA_BF16: return dw_gemm_simt_t<__nv_bfloat16>(g);
    }
    return XMA_ERR_BAD_DTYPE;
}

}  // namespace xma
