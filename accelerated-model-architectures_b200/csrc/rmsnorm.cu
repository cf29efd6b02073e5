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
#include "sm100_common.cuh"

#include <initializer_list>

namespace xma {

constexpr int RN_THREADS = 256;

template <int NT = RN_THREADS>
__device__ __forceinline__ float block_sum(float v, float* smem) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();  // smem may still be read by the previous reduction
    if (lane == 0) smem[warp] = v;
    __syncthreads();
    float t = (lane < NT / 32) ? smem[lane] : 0.0f;
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

// ---- backward, rows staged in shared memory by bulk asynchronous copies ----------------------------------------
// The register-cached kernel above keeps at most one row per CTA in flight and stalls on it at every row boundary
// (request, reduce, emit, request ...): 0.54-0.70 of the copy bandwidth. Here one thread asks the copy engine for
// whole rows (cp.async.bulk, one copy per stream of the row, completion counted in bytes on an mbarrier) STAGES - 1
// rows ahead, so that (STAGES - 1) * streams * row bytes per CTA are on their way while the CTA works on a row
// that is already in shared memory. Requirements (checked by the launcher): 128-bit rows, a row of at most 16 KiB,
// at most 1024 packets per row. Weight packets and the weight-gradient sums of a thread's columns stay in
// registers for the whole kernel.
// A wait that runs out of time (1 s) does not end the kernel and leaves no result undefined: from then on the CTA
// fills its stage with ordinary loads instead of waiting for the copy engine.
constexpr int RNB_MAX_STAGES = 4;
constexpr int RNB_CTAS_PER_SM = 2;
constexpr int RNB_MAX_ROW_BYTES = 16384;
constexpr unsigned long long RNB_WAIT_NS = 1000000000ull;

__device__ __forceinline__ void bulk_load_row(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 :
                 : "r"(tc::smem_u32(smem_dst)), "l"(gsrc), "r"(bytes), "r"(tc::smem_u32(bar))
                 : "memory");
}

__device__ __forceinline__ bool rnb_wait(uint64_t* bar, uint32_t parity, volatile int* gave_up) {
    if (tc::mbar_try_wait(bar, parity)) return true;
    const unsigned long long t0 = tc::globaltimer_ns();
    uint32_t spins = 0;
    while (!tc::mbar_try_wait(bar, parity)) {
        if ((++spins & 0x3ffu) == 0u) {
            if (*gave_up) return false;
            if (tc::globaltimer_ns() - t0 > RNB_WAIT_NS) {
                *gave_up = 1;
                return false;
            }
        }
    }
    return true;
}

template <typename T, int IPT, int NT>
__global__ void __launch_bounds__(NT, RNB_CTAS_PER_SM)
rmsnorm_bwd_bulk_kernel(const T* __restrict__ xr, int64_t xr_stride, const T* __restrict__ w,
                        const T* __restrict__ dy, int64_t dy_stride, const T* __restrict__ dxr, int64_t dxr_stride,
                        const float* __restrict__ s, T* __restrict__ dx, int64_t dx_stride, T* __restrict__ dr,
                        int64_t dr_stride, float* __restrict__ dw_partial, int64_t rows, int cols, int stages,
                        float eps, float multiplier) {
    using V = Vec16<T>;
    constexpr int N = V::N;
    extern __shared__ __align__(128) unsigned char rnb_smem[];
    __shared__ float red[NT / 32];
    __shared__ int gave_up;
    uint64_t* bars = reinterpret_cast<uint64_t*>(rnb_smem);  // [RNB_MAX_STAGES], 128 bytes reserved
    const int items = cols / N;
    const uint32_t row_bytes = static_cast<uint32_t>(cols) * sizeof(T);
    const int streams = dxr ? 3 : 2;
    unsigned char* stage0 = rnb_smem + 128;
    const uint32_t stage_bytes = streams * row_bytes;
    const float inv_cols = 1.0f / static_cast<float>(cols);
    const int tid = threadIdx.x;

    if (tid == 0) {
        gave_up = 0;
        for (int i = 0; i < stages; ++i) tc::mbar_init(&bars[i], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    uint32_t pending = 0, pending_parity = 0;  // thread 0: stages with a copy requested and not yet waited for
    auto request = [&](int64_t row, int j) {   // thread 0 only; j = the CTA's running row number
        const int st = j % stages;
        unsigned char* dst = stage0 + static_cast<size_t>(st) * stage_bytes;
        tc::mbar_expect_tx(&bars[st], stage_bytes);
        bulk_load_row(dst, xr + row * xr_stride, row_bytes, &bars[st]);
        bulk_load_row(dst + row_bytes, dy + row * dy_stride, row_bytes, &bars[st]);
        if (dxr) bulk_load_row(dst + 2 * row_bytes, dxr + row * dxr_stride, row_bytes, &bars[st]);
        pending |= 1u << st;
        pending_parity = (pending_parity & ~(1u << st)) | (static_cast<uint32_t>((j / stages) & 1) << st);
    };
    if (tid == 0) {
        int j = 0;
        for (int64_t row = blockIdx.x; row < rows && j < stages - 1; row += gridDim.x, ++j) request(row, j);
    }

    V cw[IPT];
    float acc[IPT][N];
#pragma unroll
    for (int k = 0; k < IPT; ++k) {
        const int i = tid + k * NT;
        if (w && i < items) cw[k] = load16(w + i * N);
#pragma unroll
        for (int e = 0; e < N; ++e) acc[k][e] = 0.0f;
    }

    // the stored 1/rms of the rows two and one step ahead: read directly it would put one DRAM latency under load
    // (microseconds, with every SM streaming) into each row's chain of dependent steps
    const int64_t step = gridDim.x;
    float s_now = 0.0f, s_next = 0.0f;
    if (s) {
        if (blockIdx.x < rows) s_now = s[blockIdx.x];
        if (blockIdx.x + step < rows) s_next = s[blockIdx.x + step];
    }
    bool bulk = true;  // the same in every thread of the CTA
    int j = 0;
    for (int64_t row = blockIdx.x; row < rows; row += gridDim.x, ++j) {
        const float s_row = s_now;
        s_now = s_next;
        if (s && row + 2 * step < rows) s_next = s[row + 2 * step];
        const int st = j % stages;
        unsigned char* base = stage0 + static_cast<size_t>(st) * stage_bytes;
        if (bulk && rnb_wait(&bars[st], (j / stages) & 1, &gave_up)) pending &= ~(1u << st);
        __syncthreads();  // every thread is done with the previous row (its stage is free), `gave_up` is settled
        if (bulk && gave_up) bulk = false;
        if (!bulk) {
            for (int i = tid; i < items; i += NT) {
                reinterpret_cast<V*>(base)[i] = load16(xr + row * xr_stride + i * N);
                reinterpret_cast<V*>(base + row_bytes)[i] = load16(dy + row * dy_stride + i * N);
                if (dxr) reinterpret_cast<V*>(base + 2 * row_bytes)[i] = load16(dxr + row * dxr_stride + i * N);
            }
            __syncthreads();
        } else if (tid == 0) {
            const int64_t ahead = row + static_cast<int64_t>(stages - 1) * gridDim.x;
            if (ahead < rows) request(ahead, j + stages - 1);
        }
        const V* sx = reinterpret_cast<const V*>(base);
        const V* sg = reinterpret_cast<const V*>(base + row_bytes);
        const V* se = reinterpret_cast<const V*>(base + 2 * row_bytes);

        float rstd;
        if (s) {
            rstd = s_row;
        } else {
            float sumsq = 0.0f;
#pragma unroll
            for (int k = 0; k < IPT; ++k) {
                const int i = tid + k * NT;
                if (i < items) {
                    float xv[N];
                    vec_to_f32(sx[i], xv);
#pragma unroll
                    for (int e = 0; e < N; ++e) sumsq += xv[e] * xv[e];
                }
            }
            rstd = rsqrtf(block_sum<NT>(sumsq, red) * inv_cols + eps);
        }
        // pass 1: dot = sum g * z with z = xr * rstd, g = dy * weight; d weight += dy * z. With at most 16 elements
        // per thread z and g stay in registers for pass 2 (a third of the kernel's instructions are conversions
        // and the 16-bit variants run close to the issue limit of the SM, not only to that of HBM).
        constexpr bool KEEP = sizeof(T) == 2 && IPT * N <= 16;  // fp32 has no conversions to save and measured slower with it
        float zk[KEEP ? IPT : 1][N], gk[KEEP ? IPT : 1][N];
        float dot = 0.0f;
#pragma unroll
        for (int k = 0; k < IPT; ++k) {
            const int i = tid + k * NT;
            if (i < items) {
                float xv[N], gv[N], wv[N];
                vec_to_f32(sx[i], xv);
                vec_to_f32(sg[i], gv);
                if (w) vec_to_f32(cw[k], wv);
#pragma unroll
                for (int e = 0; e < N; ++e) {
                    const float z = xv[e] * rstd;
                    acc[k][e] = fmaf(gv[e], z, acc[k][e]);
                    const float g = w ? gv[e] * wv[e] : gv[e];
                    dot = fmaf(g, z, dot);
                    if (KEEP) {
                        zk[k][e] = z;
                        gk[k][e] = g;
                    }
                }
            }
        }
        const float c = block_sum<NT>(dot, red) * inv_cols;
        const float neg_c = -c;
        const bool scaled = multiplier != 1.0f;
        // pass 2: d = (g - z * c) * rstd + d(xr)
#pragma unroll
        for (int k = 0; k < IPT; ++k) {
            const int i = tid + k * NT;
            if (i < items) {
                float ev[N], d[N];
                if (dxr) vec_to_f32(se[i], ev);
                if (KEEP) {
#pragma unroll
                    for (int e = 0; e < N; ++e) d[e] = fmaf(zk[k][e], neg_c, gk[k][e]);
                } else {
                    float xv[N], gv[N], wv[N];
                    vec_to_f32(sx[i], xv);
                    vec_to_f32(sg[i], gv);
                    if (w) vec_to_f32(cw[k], wv);
#pragma unroll
                    for (int e = 0; e < N; ++e) d[e] = fmaf(xv[e] * rstd, neg_c, w ? gv[e] * wv[e] : gv[e]);
                }
#pragma unroll
                for (int e = 0; e < N; ++e) d[e] = dxr ? fmaf(d[e], rstd, ev[e]) : d[e] * rstd;
                V q;
                vec_from_f32(d, q);
                if (dr) store16(dr + row * dr_stride + i * N, q);
                if (scaled) {
#pragma unroll
                    for (int e = 0; e < N; ++e) d[e] *= multiplier;
                    vec_from_f32(d, q);
                }
                store16(dx + row * dx_stride + i * N, q);
            }
        }
    }
    if (dw_partial) {
        float* my_dw = dw_partial + static_cast<int64_t>(blockIdx.x) * cols;
#pragma unroll
        for (int k = 0; k < IPT; ++k) {
            const int i = tid + k * NT;
            if (i < items) {
#pragma unroll
                for (int e = 0; e < N; e += 4)
                    *reinterpret_cast<float4*>(my_dw + i * N + e) =
                        make_float4(acc[k][e], acc[k][e + 1], acc[k][e + 2], acc[k][e + 3]);
            }
        }
    }
    // copies that were requested and never waited for (only after a wait gave up): one more bounded wait each, so
    // that the CTA does not leave while the copy engine may still write into its shared memory
    if (tid == 0 && pending) {
        for (int st = 0; st < stages; ++st)
            if (pending & (1u << st)) {
                int fresh = 0;
                rnb_wait(&bars[st], (pending_parity >> st) & 1u, &fresh);
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

// Shared memory of the bulk-copy backward: as many CTAs per SM (at most RNB_CTAS_PER_SM) as still keep 64 KiB of
// copies in flight per SM; with fewer bytes than that whatever keeps the most.
struct BulkPlan {
    int stages = 0, ctas_per_sm = 0, smem_bytes = 0;
};

static BulkPlan rn_bulk_plan(int64_t row_bytes, int streams) {
    BulkPlan best;
    if (row_bytes <= 0 || row_bytes > RNB_MAX_ROW_BYTES || row_bytes % 16) return best;
    const int64_t stage = streams * row_bytes;
    int64_t best_flight = -1;
    for (int ctas = RNB_CTAS_PER_SM; ctas >= 1; --ctas) {
        const int64_t room = (227 * 1024) / ctas - 1024 /*reserved per CTA*/ - 128 /*barriers*/ - 64 /*static*/;
        int64_t stages = room / stage;
        if (stages > RNB_MAX_STAGES) stages = RNB_MAX_STAGES;
        if (stages < 2) continue;
        const int64_t flight = ctas * (stages - 1) * stage;
        const bool enough = flight >= 64 * 1024;
        if (flight > best_flight) {
            best_flight = flight;
            best.stages = static_cast<int>(stages);
            best.ctas_per_sm = ctas;
            best.smem_bytes = static_cast<int>(128 + stages * stage);
        }
        if (enough) break;
    }
    return best;
}

// XMA_B200_RMSNORM_BULK=0 keeps the backward on the register-cached kernel (for comparisons).
static bool rn_bulk_enabled() {
    static const bool on = [] {
        const char* e = std::getenv("XMA_B200_RMSNORM_BULK");
        return !(e && e[0] == '0');
    }();
    return on;
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
    const bool vec = rn_vec_ok<T>(cols, {xrs, dys, dxr ? dxrs : 0, dxs, dr ? drs : 0}, {xr, w, dy, dxr, dx, dr});
    if (vec && rn_bulk_enabled() && is_aligned16(dw_partial)) {
        const int64_t items = cols / Vec16<T>::N;
        const BulkPlan plan = rn_bulk_plan(cols * static_cast<int64_t>(sizeof(T)), dxr ? 3 : 2);
        if (plan.stages >= 2 && items <= 1024) {
            int g = static_cast<int>(rows < static_cast<int64_t>(num_sms()) * plan.ctas_per_sm
                                         ? rows
                                         : static_cast<int64_t>(num_sms()) * plan.ctas_per_sm);
            if (dw_partial) {
                // `grid` is the number of partial rows the caller sums; the CTAs of this kernel fill the first g
                if (g > grid) g = grid;
                if (g < grid)
                    XMA_CUDA_TRY(cudaMemsetAsync(dw_partial + static_cast<int64_t>(g) * cols, 0,
                                                 sizeof(float) * static_cast<size_t>(grid - g) * cols, st));
            }
#define XMA_RNB_LAUNCH(IPT, NT)                                                                                     \
    do {                                                                                                            \
        auto kernel = rmsnorm_bwd_bulk_kernel<T, IPT, NT>;                                                          \
        XMA_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, plan.smem_bytes));   \
        kernel<<<g, NT, plan.smem_bytes, st>>>(xp, xrs, wp, dyp, dys, dxrp, dxrs, s, dxp, dxs, drp, drs, dw_partial, \
                                               rows, static_cast<int>(cols), plan.stages, eps, multiplier);         \
    } while (0)
            if (items <= 256) XMA_RNB_LAUNCH(1, 256);
            else if (items <= 512) XMA_RNB_LAUNCH(2, 256);
            else XMA_RNB_LAUNCH(4, 256);
#undef XMA_RNB_LAUNCH
            return static_cast<int>(cudaGetLastError());
        }
    }
    if (vec) {
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
