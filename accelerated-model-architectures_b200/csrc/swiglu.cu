// Stand-alone SwiGLU kernels behind xma.functional.swiglu / swiglu_packed
// (xma/functional/swiglu/__init__.py:39-87; math as in swiglu/torch_implementation.py:9-30):
//   y  = up * gate * sigmoid(gate)                       computed in fp32, rounded once
//   dg = dy * up * sigmoid(gate) * (1 + gate * (1 - sigmoid(gate)))
//   du = dy * gate * sigmoid(gate)
// The packed form reads gate/up interleaved along the last dimension (g,u,g,u,...).
// Inputs may be row-strided views (e.g. the two halves of `chunk(2, -1)`), so no copy is needed.
// HBM-bound: 128-bit accesses whenever widths, strides and base addresses allow, scalar otherwise.
#include "gemm_internal.h"

#include <initializer_list>

namespace xma {

constexpr int EW_THREADS = 256;

// Logistic function: exact (expf, IEEE division) for fp32 and fp16 tensors; for bf16 tensors the hardware
// ex2 / rcp approximations (a few ulp in fp32, three orders of magnitude below the rounding of the bf16 result),
// which keeps the kernel on the memory roof: with 8 elements per 128-bit packet the exact form is issue-bound.
// fp16 keeps the exact form because its results are compared with absolute tolerances of one fp16 ulp, where a
// last-bit difference in fp32 can flip the rounding.
template <typename T>
__device__ __forceinline__ float sigmoid_for(float x) {
    if (sizeof(T) == 4 || TypeInfo<T>::code == XMA_F16) return sigmoid_f32(x);
    return __fdividef(1.0f, 1.0f + __expf(-x));
}

template <typename T>
__device__ __forceinline__ float swiglu_f(float g, float u) {
    return u * g * sigmoid_for<T>(g);
}

template <typename T>
__device__ __forceinline__ void swiglu_b(float g, float u, float dy, float& dg, float& du) {
    const float s = sigmoid_for<T>(g);
    dg = dy * u * s * (1.0f + g * (1.0f - s));
    du = dy * g * s;
}

// Work items (128-bit packets, or single elements on the scalar path) are numbered row-major; a thread takes
// EW_UNROLL of them per iteration, all loads issued before the first use. Index arithmetic is 32-bit whenever
// the item count allows (a 64-bit division per packet costs more than the packet's math).
constexpr int EW_UNROLL = 2;

template <typename I>
struct ItemIndex {
    I cv;
    __device__ __forceinline__ void split(int64_t i, int64_t& r, int64_t& c) const {
        const I q = static_cast<I>(i) / cv;
        r = static_cast<int64_t>(q);
        c = static_cast<int64_t>(static_cast<I>(i) - q * cv);
    }
};

#define XMA_EW_LOOP_BEGIN                                                                                  \
    constexpr int V = VEC ? Vec16<T>::N : 1;                                                              \
    const ItemIndex<I> index{static_cast<I>(cols / V)};                                                   \
    const int64_t total = rows * (cols / V);                                                              \
    const int64_t step = static_cast<int64_t>(gridDim.x) * EW_THREADS;                                    \
    for (int64_t i0 = static_cast<int64_t>(blockIdx.x) * EW_THREADS + threadIdx.x; i0 < total;            \
         i0 += step * EW_UNROLL) {                                                                        \
        int64_t r[EW_UNROLL], c[EW_UNROLL];                                                               \
        bool on[EW_UNROLL];                                                                               \
        _Pragma("unroll") for (int k = 0; k < EW_UNROLL; ++k) {                                           \
            const int64_t i = i0 + k * step;                                                              \
            on[k] = i < total;                                                                            \
            index.split(on[k] ? i : 0, r[k], c[k]);                                                       \
            c[k] *= V;                                                                                    \
        }
#define XMA_EW_LOOP_END }

template <typename T, bool VEC, typename I>
__global__ void __launch_bounds__(EW_THREADS)
swiglu_fwd_kernel(const T* __restrict__ g, int64_t g_stride, const T* __restrict__ u, int64_t u_stride,
                  T* __restrict__ y, int64_t y_stride, int64_t rows, int64_t cols) {
    XMA_EW_LOOP_BEGIN
    if (VEC) {
        Vec16<T> a[EW_UNROLL], b[EW_UNROLL];
#pragma unroll
        for (int k = 0; k < EW_UNROLL; ++k)
            if (on[k]) {
                a[k] = load16_stream(g + r[k] * g_stride + c[k]);
                b[k] = load16_stream(u + r[k] * u_stride + c[k]);
            }
#pragma unroll
        for (int k = 0; k < EW_UNROLL; ++k)
            if (on[k]) {
                constexpr int N = Vec16<T>::N;
                float af[N], bf[N], of[N];
                vec_to_f32(a[k], af);
                vec_to_f32(b[k], bf);
#pragma unroll
                for (int j = 0; j < N; ++j) of[j] = swiglu_f<T>(af[j], bf[j]);
                Vec16<T> o;
                vec_from_f32(of, o);
                store16_stream(y + r[k] * y_stride + c[k], o);
            }
    } else {
#pragma unroll
        for (int k = 0; k < EW_UNROLL; ++k)
            if (on[k])
                y[r[k] * y_stride + c[k]] = from_f32<T>(
                    swiglu_f<T>(to_f32(g[r[k] * g_stride + c[k]]), to_f32(u[r[k] * u_stride + c[k]])));
    }
    XMA_EW_LOOP_END
}

template <typename T, bool VEC, typename I>
__global__ void __launch_bounds__(EW_THREADS)
swiglu_bwd_kernel(const T* __restrict__ g, int64_t g_stride, const T* __restrict__ u, int64_t u_stride,
                  const T* __restrict__ dy, int64_t dy_stride, T* __restrict__ dg, int64_t dg_stride,
                  T* __restrict__ du, int64_t du_stride, int64_t rows, int64_t cols) {
    XMA_EW_LOOP_BEGIN
    if (VEC) {
        Vec16<T> a[EW_UNROLL], b[EW_UNROLL], d[EW_UNROLL];
#pragma unroll
        for (int k = 0; k < EW_UNROLL; ++k)
            if (on[k]) {
                a[k] = load16_stream(g + r[k] * g_stride + c[k]);
                b[k] = load16_stream(u + r[k] * u_stride + c[k]);
                d[k] = load16_stream(dy + r[k] * dy_stride + c[k]);
            }
#pragma unroll
        for (int k = 0; k < EW_UNROLL; ++k)
            if (on[k]) {
                constexpr int N = Vec16<T>::N;
                float af[N], bf[N], df[N], gf[N], uf[N];
                vec_to_f32(a[k], af);
                vec_to_f32(b[k], bf);
                vec_to_f32(d[k], df);
#pragma unroll
                for (int j = 0; j < N; ++j) swiglu_b<T>(af[j], bf[j], df[j], gf[j], uf[j]);
                Vec16<T> og, ou;
                vec_from_f32(gf, og);
                vec_from_f32(uf, ou);
                store16_stream(dg + r[k] * dg_stride + c[k], og);
                store16_stream(du + r[k] * du_stride + c[k], ou);
            }
    } else {
#pragma unroll
        for (int k = 0; k < EW_UNROLL; ++k)
            if (on[k]) {
                float x, z;
                swiglu_b<T>(to_f32(g[r[k] * g_stride + c[k]]), to_f32(u[r[k] * u_stride + c[k]]),
                            to_f32(dy[r[k] * dy_stride + c[k]]), x, z);
                dg[r[k] * dg_stride + c[k]] = from_f32<T>(x);
                du[r[k] * du_stride + c[k]] = from_f32<T>(z);
            }
    }
    XMA_EW_LOOP_END
}

// Packed: x[r, 2c] = gate, x[r, 2c+1] = up; y[r, c]. `cols` is the width of y.
template <typename T, bool VEC, typename I>
__global__ void __launch_bounds__(EW_THREADS)
swiglu_packed_fwd_kernel(const T* __restrict__ x, int64_t x_stride, T* __restrict__ y, int64_t y_stride,
                         int64_t rows, int64_t cols) {
    XMA_EW_LOOP_BEGIN
    if (VEC) {
        constexpr int N = Vec16<T>::N;
        Vec16<T> a[EW_UNROLL], b[EW_UNROLL];
#pragma unroll
        for (int k = 0; k < EW_UNROLL; ++k)
            if (on[k]) {
                a[k] = load16_stream(x + r[k] * x_stride + 2 * c[k]);
                b[k] = load16_stream(x + r[k] * x_stride + 2 * c[k] + N);
            }
#pragma unroll
        for (int k = 0; k < EW_UNROLL; ++k)
            if (on[k]) {
                float af[N], bf[N], of[N];
                vec_to_f32(a[k], af);
                vec_to_f32(b[k], bf);
#pragma unroll
                for (int j = 0; j < N / 2; ++j) {
                    of[j] = swiglu_f<T>(af[2 * j], af[2 * j + 1]);
                    of[j + N / 2] = swiglu_f<T>(bf[2 * j], bf[2 * j + 1]);
                }
                Vec16<T> o;
                vec_from_f32(of, o);
                store16_stream(y + r[k] * y_stride + c[k], o);
            }
    } else {
#pragma unroll
        for (int k = 0; k < EW_UNROLL; ++k)
            if (on[k])
                y[r[k] * y_stride + c[k]] = from_f32<T>(swiglu_f<T>(to_f32(x[r[k] * x_stride + 2 * c[k]]),
                                                                    to_f32(x[r[k] * x_stride + 2 * c[k] + 1])));
    }
    XMA_EW_LOOP_END
}

template <typename T, bool VEC, typename I>
__global__ void __launch_bounds__(EW_THREADS)
swiglu_packed_bwd_kernel(const T* __restrict__ x, int64_t x_stride, const T* __restrict__ dy, int64_t dy_stride,
                         T* __restrict__ dx, int64_t dx_stride, int64_t rows, int64_t cols) {
    XMA_EW_LOOP_BEGIN
    if (VEC) {
        constexpr int N = Vec16<T>::N;
        Vec16<T> a[EW_UNROLL], b[EW_UNROLL], d[EW_UNROLL];
#pragma unroll
        for (int k = 0; k < EW_UNROLL; ++k)
            if (on[k]) {
                a[k] = load16_stream(x + r[k] * x_stride + 2 * c[k]);
                b[k] = load16_stream(x + r[k] * x_stride + 2 * c[k] + N);
                d[k] = load16_stream(dy + r[k] * dy_stride + c[k]);
            }
#pragma unroll
        for (int k = 0; k < EW_UNROLL; ++k)
            if (on[k]) {
                float af[N], bf[N], df[N], pa[N], pb[N];
                vec_to_f32(a[k], af);
                vec_to_f32(b[k], bf);
                vec_to_f32(d[k], df);
#pragma unroll
                for (int j = 0; j < N / 2; ++j) {
                    swiglu_b<T>(af[2 * j], af[2 * j + 1], df[j], pa[2 * j], pa[2 * j + 1]);
                    swiglu_b<T>(bf[2 * j], bf[2 * j + 1], df[j + N / 2], pb[2 * j], pb[2 * j + 1]);
                }
                Vec16<T> oa, ob;
                vec_from_f32(pa, oa);
                vec_from_f32(pb, ob);
                store16_stream(dx + r[k] * dx_stride + 2 * c[k], oa);
                store16_stream(dx + r[k] * dx_stride + 2 * c[k] + N, ob);
            }
    } else {
#pragma unroll
        for (int k = 0; k < EW_UNROLL; ++k)
            if (on[k]) {
                float p, q;
                swiglu_b<T>(to_f32(x[r[k] * x_stride + 2 * c[k]]), to_f32(x[r[k] * x_stride + 2 * c[k] + 1]),
                            to_f32(dy[r[k] * dy_stride + c[k]]), p, q);
                dx[r[k] * dx_stride + 2 * c[k]] = from_f32<T>(p);
                dx[r[k] * dx_stride + 2 * c[k] + 1] = from_f32<T>(q);
            }
    }
    XMA_EW_LOOP_END
}

static int ew_grid(int64_t work_items) {
    int64_t want = ceil_div(work_items, EW_THREADS * EW_UNROLL);
    int64_t cap = static_cast<int64_t>(num_sms()) * 16;
    return static_cast<int>(want < 1 ? 1 : (want > cap ? cap : want));
}

// 32-bit item arithmetic when every item index (and one unrolled step beyond the end) fits
#define XMA_EW_LAUNCH(kernel, vec, items, stream, ...)                                                  \
    do {                                                                                                \
        const int64_t n_items = (items);                                                                \
        if (n_items < (int64_t{1} << 31))                                                               \
            kernel<T, vec, uint32_t><<<ew_grid(n_items), EW_THREADS, 0, stream>>>(__VA_ARGS__);         \
        else                                                                                            \
            kernel<T, vec, uint64_t><<<ew_grid(n_items), EW_THREADS, 0, stream>>>(__VA_ARGS__);         \
    } while (0)

template <typename T>
static bool vec_ok(int64_t cols, std::initializer_list<int64_t> strides, std::initializer_list<const void*> ptrs) {
    constexpr int V = Vec16<T>::N;
    if (cols % V) return false;
    for (int64_t s : strides)
        if (s % V) return false;
    for (const void* p : ptrs)
        if (!is_aligned16(p)) return false;
    return true;
}

template <typename T>
static int swiglu_fwd_impl(const void* g, int64_t gs, const void* u, int64_t us, void* y, int64_t ys, int64_t rows,
                           int64_t cols, cudaStream_t st) {
    const T* gp = static_cast<const T*>(g);
    const T* up = static_cast<const T*>(u);
    T* yp = static_cast<T*>(y);
    if (vec_ok<T>(cols, {gs, us, ys}, {g, u, y}))
        XMA_EW_LAUNCH(swiglu_fwd_kernel, true, rows * cols / Vec16<T>::N, st, gp, gs, up, us, yp, ys, rows, cols);
    else
        XMA_EW_LAUNCH(swiglu_fwd_kernel, false, rows * cols, st, gp, gs, up, us, yp, ys, rows, cols);
    return static_cast<int>(cudaGetLastError());
}

template <typename T>
static int swiglu_bwd_impl(const void* g, int64_t gs, const void* u, int64_t us, const void* dy, int64_t dys,
                           void* dg, int64_t dgs, void* du, int64_t dus, int64_t rows, int64_t cols,
                           cudaStream_t st) {
    const T* gp = static_cast<const T*>(g);
    const T* up = static_cast<const T*>(u);
    const T* dyp = static_cast<const T*>(dy);
    T* dgp = static_cast<T*>(dg);
    T* dup = static_cast<T*>(du);
    if (vec_ok<T>(cols, {gs, us, dys, dgs, dus}, {g, u, dy, dg, du}))
        XMA_EW_LAUNCH(swiglu_bwd_kernel, true, rows * cols / Vec16<T>::N, st, gp, gs, up, us, dyp, dys, dgp, dgs, dup, dus, rows, cols);
    else
        XMA_EW_LAUNCH(swiglu_bwd_kernel, false, rows * cols, st, gp, gs, up, us, dyp, dys, dgp, dgs, dup, dus, rows, cols);
    return static_cast<int>(cudaGetLastError());
}

template <typename T>
static int swiglu_packed_fwd_impl(const void* x, int64_t xs, void* y, int64_t ys, int64_t rows, int64_t cols,
                                  cudaStream_t st) {
    const T* xp = static_cast<const T*>(x);
    T* yp = static_cast<T*>(y);
    if (vec_ok<T>(cols, {xs, ys}, {x, y}))
        XMA_EW_LAUNCH(swiglu_packed_fwd_kernel, true, rows * cols / Vec16<T>::N, st, xp, xs, yp, ys, rows, cols);
    else
        XMA_EW_LAUNCH(swiglu_packed_fwd_kernel, false, rows * cols, st, xp, xs, yp, ys, rows, cols);
    return static_cast<int>(cudaGetLastError());
}

template <typename T>
static int swiglu_packed_bwd_impl(const void* x, int64_t xs, const void* dy, int64_t dys, void* dx, int64_t dxs,
                                  int64_t rows, int64_t cols, cudaStream_t st) {
    const T* xp = static_cast<const T*>(x);
    const T* dyp = static_cast<const T*>(dy);
    T* dxp = static_cast<T*>(dx);
    if (vec_ok<T>(cols, {xs, dys, dxs}, {x, dy, dx}))
        XMA_EW_LAUNCH(swiglu_packed_bwd_kernel, true, rows * cols / Vec16<T>::N, st, xp, xs, dyp, dys, dxp, dxs, rows, cols);
    else
        XMA_EW_LAUNCH(swiglu_packed_bwd_kernel, false, rows * cols, st, xp, xs, dyp, dys, dxp, dxs, rows, cols);
    return static_cast<int>(cudaGetLastError());
}

}  // namespace xma

#define XMA_DISPATCH_FLOAT(dtype, CALL)             \
    switch (dtype) {                                \
        case XMA_F32: { using T = float; return CALL; }            \
        case XMA_F16: { using T = __half; return CALL; }           \
        case XMA_BF16: { using T = __nv_bfloat16; return CALL; }   \
        default: return XMA_ERR_BAD_DTYPE;          \
    }

namespace xma {

int swiglu_fwd_launch(const void* g, int64_t gs, const void* u, int64_t us, void* y, int64_t ys, int dtype,
                      int64_t rows, int64_t cols, cudaStream_t st) {
    if (rows <= 0 || cols <= 0) return XMA_OK;
    XMA_DISPATCH_FLOAT(dtype, swiglu_fwd_impl<T>(g, gs, u, us, y, ys, rows, cols, st));
}

int swiglu_bwd_launch(const void* g, int64_t gs, const void* u, int64_t us, const void* dy, int64_t dys, void* dg,
                      int64_t dgs, void* du, int64_t dus, int dtype, int64_t rows, int64_t cols, cudaStream_t st) {
    if (rows <= 0 || cols <= 0) return XMA_OK;
    XMA_DISPATCH_FLOAT(dtype, swiglu_bwd_impl<T>(g, gs, u, us, dy, dys, dg, dgs, du, dus, rows, cols, st));
}

}  // namespace xma

extern "C" {

int xma_b200_swiglu_fwd(const void* gate, int64_t gate_row_stride, const void* up, int64_t up_row_stride, void* y,
                        int64_t y_row_stride, int dtype, int64_t rows, int64_t cols, cudaStream_t stream) {
    if (rows < 0 || cols < 0) return XMA_ERR_BAD_SHAPE;
    if (rows == 0 || cols == 0) return XMA_OK;
    if (!gate || !up || !y) return XMA_ERR_NULL_POINTER;
    XMA_DISPATCH_FLOAT(dtype, xma::swiglu_fwd_impl<T>(gate, gate_row_stride, up, up_row_stride, y, y_row_stride,
                                                      rows, cols, stream));
}

int xma_b200_swiglu_bwd(const void* gate, int64_t gate_row_stride, const void* up, int64_t up_row_stride,
                        const void* dy, int64_t dy_row_stride, void* dgate, int64_t dgate_row_stride, void* dup,
                        int64_t dup_row_stride, int dtype, int64_t rows, int64_t cols, cudaStream_t stream) {
    if (rows < 0 || cols < 0) return XMA_ERR_BAD_SHAPE;
    if (rows == 0 || cols == 0) return XMA_OK;
    if (!gate || !up || !dy || !dgate || !dup) return XMA_ERR_NULL_POINTER;
    XMA_DISPATCH_FLOAT(dtype,
                       xma::swiglu_bwd_impl<T>(gate, gate_row_stride, up, up_row_stride, dy, dy_row_stride, dgate,
                                               dgate_row_stride, dup, dup_row_stride, rows, cols, stream));
}

int xma_b200_swiglu_packed_fwd(const void* x, int64_t x_row_stride, void* y, int64_t y_row_stride, int dtype,
                               int64_t rows, int64_t out_cols, cudaStream_t stream) {
    if (rows < 0 || out_cols < 0) return XMA_ERR_BAD_SHAPE;
    if (rows == 0 || out_cols == 0) return XMA_OK;
    if (!x || !y) return XMA_ERR_NULL_POINTER;
    XMA_DISPATCH_FLOAT(dtype, xma::swiglu_packed_fwd_impl<T>(x, x_row_stride, y, y_row_stride, rows, out_cols, stream));
}

int xma_b200_swiglu_packed_bwd(const void* x, int64_t x_row_stride, const void* dy, int64_t dy_row_stride, void* dx,
                               int64_t dx_row_stride, int dtype, int64_t rows, int64_t out_cols,
                               cudaStream_t stream) {
    if (rows < 0 || out_cols < 0) return XMA_ERR_BAD_SHAPE;
    if (rows == 0 || out_cols == 0) return XMA_OK;
    if (!x || !dy || !dx) return XMA_ERR_NULL_POINTER;
    XMA_DISPATCH_FLOAT(dtype, xma::swiglu_packed_bwd_impl<T>(x, x_row_stride, dy, dy_row_stride, dx, dx_row_stride,
                                                             rows, out_cols, stream));
}

}  // extern "C"
