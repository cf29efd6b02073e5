// fused_residual_add_rmsnorm: the step in front of the MoE layer in a transformer block
// (xma/functional/fused_residual_add_rmsnorm/__init__.py:27-83; math as in torch_implementation.py:9-27,
// kernels replaced: triton_implementation/forward.py and backward.py):
//   v  = x * multiplier + residual          (each term optional)      -> new residual stream `xr`
//   y  = v * rsqrt(mean(v^2) + eps) * weight
// and its backward
//   z = xr * rstd,  g = dy * weight,  d = (g - z * mean(g * z)) * rstd + d(xr)
//   d residual = d,  d x = d * multiplier,  d weight = sum over rows of dy * z.
// HBM-bound: one CTA per row (grid-stride), 128-bit accesses, the row cached in registers between the
// reduction and the normalisation so that every element is read once (rows too long for the cache, and
// rows whose width or alignment rules out 128-bit accesses, are read twice; the second read hits L1/L2).
// The normalisation uses the value that is stored as `xr` (rounded to the storage type), so the backward,
// which only sees `xr`, differentiates exactly what the forward computed.
#include "common.cuh"

#include <initializer_list>

namespace xma {

constexpr int RN_THREADS = 256;

__device__ __forceinline__ float block_sum(float v, float* smem) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();  // smem may still be read by the previous reduction
    if (lane == 0) smem[warp] = v;
    __syncthreads();
    float t = (lane < RN_THREADS / 32) ? smem[lane] : 0.0f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    return t;
}

// One "item" is a 128-bit packet (VEC) or a single element. Thread t owns items t, t + 256, ...;
// the first CACHE of them stay in registers between the two passes over the row.
template <typename T, bool VEC>
struct Item {
    static constexpr int N = VEC ? Vec16<T>::N : 1;
    float v[N];
    __device__ __forceinline__ void load(const T* p) {
        if constexpr (VEC) {
            const Vec16<T> q = load16(p);
            vec_to_f32(q, v);
        } else {
            v[0] = to_f32(p[0]);
        }
    }
    __device__ __forceinline__ void store(T* p) const {
        if constexpr (VEC) {
            Vec16<T> q;
            vec_from_f32(v, q);
            store16(p, q);
        } else {
            p[0] = from_f32<T>(v[0]);
        }
    }
    __device__ __forceinline__ void round_to_storage() {
#pragma unroll
        for (int j = 0; j < N; ++j) v[j] = to_f32(from_f32<T>(v[j]));
    }
};

template <typename T, bool VEC, int CACHE>
__global__ void __launch_bounds__(RN_THREADS)
rmsnorm_fwd_kernel(const T* __restrict__ x, int64_t x_stride, const T* __restrict__ r, int64_t r_stride,
                   const T* __restrict__ w, T* __restrict__ y, int64_t y_stride, T* __restrict__ xr,
                   int64_t xr_stride, float* __restrict__ s, int64_t rows, int64_t cols, float eps, float multiplier) {
    using It = Item<T, VEC>;
    constexpr int N = It::N;
    __shared__ float red[RN_THREADS / 32];
    const int64_t items = cols / N;
    const float inv_cols = 1.0f / static_cast<float>(cols);
    for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const T* xp = x + row * x_stride;
        const T* rp = r ? r + row * r_stride : nullptr;
        T* xrp = xr ? xr + row * xr_stride : nullptr;
        It cache[CACHE > 0 ? CACHE : 1];
        // the new residual stream of one item: x * multiplier (+ residual), rounded as it is stored
        auto stream_value = [&](int64_t i, It& a) {
            a.load(xp + i * N);
#pragma unroll
            for (int j = 0; j < N; ++j) a.v[j] *= multiplier;
            if (rp) {
                It b;
                b.load(rp + i * N);
#pragma unroll
                for (int j = 0; j < N; ++j) a.v[j] += b.v[j];
            }
            a.round_to_storage();
        };
        float sumsq = 0.0f;
#pragma unroll
        for (int k = 0; k < CACHE; ++k) {
            const int64_t i = threadIdx.x + static_cast<int64_t>(k) * RN_THREADS;
            if (i < items) {
                stream_value(i, cache[k]);
                if (xrp) cache[k].store(xrp + i * N);
#pragma unroll
                for (int j = 0; j < N; ++j) sumsq += cache[k].v[j] * cache[k].v[j];
            }
        }
        for (int64_t i = threadIdx.x + static_cast<int64_t>(CACHE) * RN_THREADS; i < items; i += RN_THREADS) {
            It a;
            stream_value(i, a);
            if (xrp) a.store(xrp + i * N);
#pragma unroll
            for (int j = 0; j < N; ++j) sumsq += a.v[j] * a.v[j];
        }
        const float rstd = rsqrtf(block_sum(sumsq, red) * inv_cols + eps);
        if (s && threadIdx.x == 0) s[row] = rstd;
        T* yp = y + row * y_stride;
        auto normalise = [&](int64_t i, It& a) {
            if (w) {
                It g;
                g.load(w + i * N);
#pragma unroll
                for (int j = 0; j < N; ++j) a.v[j] = a.v[j] * rstd * g.v[j];
            } else {
#pragma unroll
                for (int j = 0; j < N; ++j) a.v[j] *= rstd;
            }
            a.store(yp + i * N);
        };
#pragma unroll
        for (int k = 0; k < CACHE; ++k) {
            const int64_t i = threadIdx.x + static_cast<int64_t>(k) * RN_THREADS;
            if (i < items) normalise(i, cache[k]);
        }
        for (int64_t i = threadIdx.x + static_cast<int64_t>(CACHE) * RN_THREADS; i < items; i += RN_THREADS) {
            It a;
            stream_value(i, a);  // second read of a long row: the same arithmetic, the same rounded value
            normalise(i, a);
        }
    }
}

// d weight: every CTA adds dy * z of its rows into row blockIdx.x of `dw_partial` [gridDim.x, cols] (fp32); the
// caller sums the partial rows. A thread always meets the same columns, so the CTA's running sums live in shared
// memory without atomics (cached items; 32 KiB at most) or in the CTA's own partial row (rows too long to cache).
// The cached items stay in registers in their storage type (a 128-bit packet is four registers, its eight
// fp32 values would be eight), and the three streams of a row (xr, dy, d xr) are all requested before the first
// use: with 114 registers and the d(xr) load issued behind the row reduction the first version kept too few
// bytes in flight (0.49 of the copy bandwidth).
template <typename T, bool VEC>
struct Raw {
    static constexpr int N = VEC ? Vec16<T>::N : 1;
    Vec16<T> q;  // only element 0 is used on the scalar path
    __device__ __forceinline__ void load(const T* p) {
        if (VEC) q = load16(p);
        else q.v[0] = p[0];
    }
    __device__ __forceinline__ float at(int j) const { return to_f32(q.v[j]); }
};

template <typename T, bool VEC, int CACHE>
__global__ void __launch_bounds__(RN_THREADS, (CACHE <= 2 ? 2 : 1))
rmsnorm_bwd_kernel(const T* __restrict__ xr, int64_t xr_stride, const T* __restrict__ w, const T* __restrict__ dy,
                   int64_t dy_stride, const T* __restrict__ dxr, int64_t dxr_stride, const float* __restrict__ s,
                   T* __restrict__ dx, int64_t dx_stride, T* __restrict__ dr, int64_t dr_stride,
                   float* __restrict__ dw_partial, int64_t rows, int64_t cols, float eps, float multiplier) {
    using It = Item<T, VEC>;
    using Rw = Raw<T, VEC>;
    constexpr int N = It::N;
    constexpr int C = CACHE > 0 ? CACHE : 1;
    __shared__ float red[RN_THREADS / 32];
    extern __shared__ float s_dw[];  // [CACHE * RN_THREADS * N] when the weight gradient is wanted
    const int64_t items = cols / N;
    const float inv_cols = 1.0f / static_cast<float>(cols);
    float* my_dw = dw_partial ? dw_partial + static_cast<int64_t>(blockIdx.x) * cols : nullptr;
    if (my_dw) {
        for (int i = threadIdx.x; i < CACHE * RN_THREADS * N; i += RN_THREADS) s_dw[i] = 0.0f;
        for (int64_t i = threadIdx.x + static_cast<int64_t>(CACHE) * RN_THREADS; i < items; i += RN_THREADS)
#pragma unroll
            for (int j = 0; j < N; ++j) my_dw[i * N + j] = 0.0f;
        // (each thread only ever touches its own entries of s_dw and of my_dw: no barrier needed)
    }

    for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const T* xp = xr + row * xr_stride;
        const T* dyp = dy + row * dy_stride;
        const T* dxrp = dxr ? dxr + row * dxr_stride : nullptr;
        Rw cx[C], cg[C], ce[C];
        // every cached packet of the row's three streams is requested here
#pragma unroll
        for (int k = 0; k < CACHE; ++k) {
            const int64_t i = threadIdx.x + static_cast<int64_t>(k) * RN_THREADS;
            if (i < items) {
                cx[k].load(xp + i * N);
                cg[k].load(dyp + i * N);
                if (dxrp) ce[k].load(dxrp + i * N);
            }
        }
        float rstd;
        if (s) {
            rstd = s[row];
        } else {
            float sumsq = 0.0f;
#pragma unroll
            for (int k = 0; k < CACHE; ++k) {
                const int64_t i = threadIdx.x + static_cast<int64_t>(k) * RN_THREADS;
                if (i < items)
#pragma unroll
                    for (int j = 0; j < N; ++j) sumsq += cx[k].at(j) * cx[k].at(j);
            }
            for (int64_t i = threadIdx.x + static_cast<int64_t>(CACHE) * RN_THREADS; i < items; i += RN_THREADS) {
                It a;
                a.load(xp + i * N);
#pragma unroll
                for (int j = 0; j < N; ++j) sumsq += a.v[j] * a.v[j];
            }
            rstd = rsqrtf(block_sum(sumsq, red) * inv_cols + eps);
        }
        // pass 1: z = xr * rstd, g = dy * weight, dot = sum g * z; d weight += dy * z
        float dot = 0.0f;
#pragma unroll
        for (int k = 0; k < CACHE; ++k) {
            const int64_t i = threadIdx.x + static_cast<int64_t>(k) * RN_THREADS;
            if (i < items) {
                It ww;
                if (w) ww.load(w + i * N);
#pragma unroll
                for (int j = 0; j < N; ++j) {
                    const float z = cx[k].at(j) * rstd, g = cg[k].at(j);
                    if (my_dw) s_dw[(k * RN_THREADS + threadIdx.x) * N + j] += g * z;
                    dot += (w ? g * ww.v[j] : g) * z;
                }
            }
        }
        for (int64_t i = threadIdx.x + static_cast<int64_t>(CACHE) * RN_THREADS; i < items; i += RN_THREADS) {
            It z, g, ww;
            z.load(xp + i * N);
            g.load(dyp + i * N);
            if (w) ww.load(w + i * N);
#pragma unroll
            for (int j = 0; j < N; ++j) {
                const float zz = z.v[j] * rstd;
                if (my_dw) my_dw[i * N + j] += g.v[j] * zz;
                dot += (w ? g.v[j] * ww.v[j] : g.v[j]) * zz;
            }
        }
        const float c = block_sum(dot, red) * inv_cols;
        // pass 2: d = (g - z * c) * rstd + d(xr)
        auto emit = [&](int64_t i, const float* z, const float* g, const float* e) {
            It d;
#pragma unroll
            for (int j = 0; j < N; ++j) d.v[j] = (g[j] - z[j] * c) * rstd + (e ? e[j] : 0.0f);
            if (dr) d.store(dr + row * dr_stride + i * N);
#pragma unroll
            for (int j = 0; j < N; ++j) d.v[j] *= multiplier;
            d.store(dx + row * dx_stride + i * N);
        };
#pragma unroll
        for (int k = 0; k < CACHE; ++k) {
            const int64_t i = threadIdx.x + static_cast<int64_t>(k) * RN_THREADS;
            if (i < items) {
                It ww;
                if (w) ww.load(w + i * N);
                float z[N], g[N], e[N];
#pragma unroll
                for (int j = 0; j < N; ++j) {
                    z[j] = cx[k].at(j) * rstd;
                    g[j] = w ? cg[k].at(j) * ww.v[j] : cg[k].at(j);
                    e[j] = dxrp ? ce[k].at(j) : 0.0f;
                }
                emit(i, z, g, dxrp ? e : nullptr);
            }
        }
        for (int64_t i = threadIdx.x + static_cast<int64_t>(CACHE) * RN_THREADS; i < items; i += RN_THREADS) {
            It z, g, e;
            z.load(xp + i * N);
            g.load(dyp + i * N);
            if (dxrp) e.load(dxrp + i * N);
#pragma unroll
            for (int j = 0; j < N; ++j) z.v[j] *= rstd;
            if (w) {
                It ww;
                ww.load(w + i * N);
#pragma unroll
                for (int j = 0; j < N; ++j) g.v[j] *= ww.v[j];
            }
            emit(i, z.v, g.v, dxrp ? e.v : nullptr);
        }
    }
    if (my_dw) {
#pragma unroll
        for (int k = 0; k < CACHE; ++k) {
            const int64_t i = threadIdx.x + static_cast<int64_t>(k) * RN_THREADS;
            if (i < items)
#pragma unroll
                for (int j = 0; j < N; ++j) my_dw[i * N + j] = s_dw[(k * RN_THREADS + threadIdx.x) * N + j];
        }
    }
}

static int rn_grid(int64_t rows) {
    const int64_t cap = static_cast<int64_t>(num_sms()) * 4;
    return static_cast<int>(rows < 1 ? 1 : (rows > cap ? cap : rows));
}

template <typename T>
static bool rn_vec_ok(int64_t cols, std::initializer_list<int64_t> strides, std::initializer_list<const void*> ptrs) {
    constexpr int V = Vec16<T>::N;
    if (cols % V) return false;
    for (int64_t st : strides)
        if (st % V) return false;
    for (const void* p : ptrs)
        if (p && !is_aligned16(p)) return false;
    return true;
}

// items per thread kept in registers: enough for the whole row when it has at most 8 * 256 items
static int cache_for(int64_t items) {
    if (items <= RN_THREADS) return 1;
    if (items <= 2 * RN_THREADS) return 2;
    if (items <= 4 * RN_THREADS) return 4;
    if (items <= 8 * RN_THREADS) return 8;
    return 0;
}

// SMEM_PER_ITEM: dynamic shared memory per cached item slot (the backward's weight-gradient sums), 0 for none
#define XMA_RN_DISPATCH(KERNEL, VEC, items, grid, SMEM_PER_ITEM, stream, ...)                                       \
    switch (cache_for(items)) {                                                                                     \
        case 1: KERNEL<T, VEC, 1><<<grid, RN_THREADS, 1 * (SMEM_PER_ITEM), stream>>>(__VA_ARGS__); break;           \
        case 2: KERNEL<T, VEC, 2><<<grid, RN_THREADS, 2 * (SMEM_PER_ITEM), stream>>>(__VA_ARGS__); break;           \
        case 4: KERNEL<T, VEC, 4><<<grid, RN_THREADS, 4 * (SMEM_PER_ITEM), stream>>>(__VA_ARGS__); break;           \
        case 8: KERNEL<T, VEC, 8><<<grid, RN_THREADS, 8 * (SMEM_PER_ITEM), stream>>>(__VA_ARGS__); break;           \
        default: KERNEL<T, VEC, 0><<<grid, RN_THREADS, 0, stream>>>(__VA_ARGS__); break;                            \
    }

template <typename T>
static int rmsnorm_fwd_impl(const void* x, int64_t xs, const void* r, int64_t rs, const void* w, void* y, int64_t ys,
                            void* xr, int64_t xrs, float* s, int64_t rows, int64_t cols, float eps, float multiplier,
                            cudaStream_t st) {
    const T* xp = static_cast<const T*>(x);
    const T* rp = static_cast<const T*>(r);
    const T* wp = static_cast<const T*>(w);
    T* yp = static_cast<T*>(y);
    T* xrp = static_cast<T*>(xr);
    const int grid = rn_grid(rows);
    if (rn_vec_ok<T>(cols, {xs, r ? rs : 0, ys, xr ? xrs : 0}, {x, r, w, y, xr})) {
        XMA_RN_DISPATCH(rmsnorm_fwd_kernel, true, cols / Vec16<T>::N, grid, 0, st, xp, xs, rp, rs, wp, yp, ys, xrp, xrs, s,
                        rows, cols, eps, multiplier)
    } else {
        XMA_RN_DISPATCH(rmsnorm_fwd_kernel, false, cols, grid, 0, st, xp, xs, rp, rs, wp, yp, ys, xrp, xrs, s, rows, cols,
                        eps, multiplier)
    }
    return static_cast<int>(cudaGetLastError());
}

template <typename T>
static int rmsnorm_bwd_impl(const void* xr, int64_t xrs, const void* w, const void* dy, int64_t dys, const void* dxr,
                            int64_t dxrs, const float* s, void* dx, int64_t dxs, void* dr, int64_t drs,
                            float* dw_partial, int grid, int64_t rows, int64_t cols, float eps, float multiplier,
                            cudaStream_t st) {
    const T* xp = static_cast<const T*>(xr);
    const T* wp = static_cast<const T*>(w);
    const T* dyp = static_cast<const T*>(dy);
    const T* dxrp = static_cast<const T*>(dxr);
    T* dxp = static_cast<T*>(dx);
    T* drp = static_cast<T*>(dr);
    if (rn_vec_ok<T>(cols, {xrs, dys, dxr ? dxrs : 0, dxs, dr ? drs : 0}, {xr, w, dy, dxr, dx, dr})) {
        XMA_RN_DISPATCH(rmsnorm_bwd_kernel, true, cols / Vec16<T>::N, grid,
                        (dw_partial ? RN_THREADS * Vec16<T>::N * sizeof(float) : 0), st, xp, xrs, wp, dyp, dys, dxrp, dxrs, s,
                        dxp, dxs, drp, drs, dw_partial, rows, cols, eps, multiplier)
    } else {
        XMA_RN_DISPATCH(rmsnorm_bwd_kernel, false, cols, grid, (dw_partial ? RN_THREADS * sizeof(float) : 0), st, xp, xrs, wp, dyp, dys, dxrp, dxrs, s, dxp, dxs, drp,
                        drs, dw_partial, rows, cols, eps, multiplier)
    }
    return static_cast<int>(cudaGetLastError());
}

}  // namespace xma

#define XMA_RN_FLOAT(dtype, CALL)                                  \
    switch (dtype) {                                               \
        case XMA_F32: { using T = float; return CALL; }            \
        case XMA_F16: { using T = __half; return CALL; }           \
        case XMA_BF16: { using T = __nv_bfloat16; return CALL; }   \
        default: return XMA_ERR_BAD_DTYPE;                         \
    }

extern "C" {

int xma_b200_rmsnorm_fwd(const void* x, int64_t x_row_stride, const void* residual, int64_t residual_row_stride,
                         const void* weight, void* y, int64_t y_row_stride, void* xr, int64_t xr_row_stride,
                         float* rstd, int dtype, int64_t rows, int64_t cols, float eps, float multiplier,
                         cudaStream_t stream) {
    if (rows < 0 || cols < 0) return XMA_ERR_BAD_SHAPE;
    if (rows == 0 || cols == 0) return XMA_OK;
    if (!x || !y) return XMA_ERR_NULL_POINTER;
    if (residual && !xr) return XMA_ERR_NULL_POINTER;  // the updated residual stream is an output then
    XMA_RN_FLOAT(dtype, xma::rmsnorm_fwd_impl<T>(x, x_row_stride, residual, residual_row_stride, weight, y,
                                                 y_row_stride, xr, xr_row_stride, rstd, rows, cols, eps, multiplier,
                                                 stream));
}

int xma_b200_rmsnorm_bwd_partial_rows(int64_t rows) { return xma::rn_grid(rows); }

int xma_b200_rmsnorm_bwd(const void* xr, int64_t xr_row_stride, const void* weight, const void* dy,
                         int64_t dy_row_stride, const void* dxr, int64_t dxr_row_stride, const float* rstd, void* dx,
                         int64_t dx_row_stride, void* dresidual, int64_t dresidual_row_stride, float* dweight_partial,
                         int partial_rows, int dtype, int64_t rows, int64_t cols, float eps, float multiplier,
                         cudaStream_t stream) {
    if (rows < 0 || cols < 0) return XMA_ERR_BAD_SHAPE;
    if (dweight_partial && partial_rows <= 0) return XMA_ERR_BAD_SHAPE;
    if (rows == 0 || cols == 0) {
        if (dweight_partial && cols > 0)
            XMA_CUDA_TRY(cudaMemsetAsync(dweight_partial, 0, sizeof(float) * partial_rows * cols, stream));
        return XMA_OK;
    }
    if (!xr || !dy || !dx) return XMA_ERR_NULL_POINTER;
    const int grid = dweight_partial ? partial_rows : xma::rn_grid(rows);
    XMA_RN_FLOAT(dtype, xma::rmsnorm_bwd_impl<T>(xr, xr_row_stride, weight, dy, dy_row_stride, dxr, dxr_row_stride, rstd,
                                                 dx, dx_row_stride, dresidual, dresidual_row_stride, dweight_partial,
                                                 grid, rows, cols, eps, multiplier, stream));
}

}  // extern "C"
