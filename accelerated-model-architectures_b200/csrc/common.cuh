// Shared helpers for the sm_100a MoE hot-path kernels: status codes, dtype codes,
// 128-bit load/store helpers and bf16/fp16 <-> fp32 conversion.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

// ---- return codes of every extern "C" entry point -------------------------------------------
// 0            : launched (asynchronously) without a host-visible error
// negative     : argument error detected on the host, nothing was launched
// positive     : cudaError_t of a failed runtime call or launch
#define XMA_OK 0
#define XMA_ERR_NULL_POINTER (-1)
#define XMA_ERR_BAD_DTYPE (-2)
#define XMA_ERR_BAD_SHAPE (-3)
#define XMA_ERR_SCRATCH_TOO_SMALL (-4)
#define XMA_ERR_UNSUPPORTED (-5)
#define XMA_ERR_MISALIGNED (-6)
#define XMA_ERR_TENSOR_MAP (-7)
#define XMA_ERR_TOO_LARGE (-8)

// ---- bits of the asynchronous device status word (int32 the caller owns, may be null) -------
#define XMA_DEV_ID_OUT_OF_RANGE 1  // an expert id / bin id outside [0, bins) was skipped
#define XMA_DEV_WAIT_TIMEOUT 2     // a bounded device-side wait gave up
#define XMA_DEV_BAD_TILE 4         // a tile table entry was inconsistent and was skipped

// ---- dtype codes ------------------------------------------------------------------------------
#define XMA_F32 0
#define XMA_F16 1
#define XMA_BF16 2
#define XMA_I32 3
#define XMA_I64 4

// Rows of the expert-sorted ("grouped") buffers are padded per expert to a multiple of this, so
// that a 128-row GEMM tile never straddles two experts and the reduction blocks of the weight
// gradient GEMMs never mix experts.
#define XMA_ROW_PAD 128

#define XMA_CUDA_TRY(expr)                         \
    do {                                           \
        cudaError_t _e = (expr);                   \
        if (_e != cudaSuccess) return (int)_e;     \
    } while (0)

namespace xma {

// Expert-parallel row maps address a row of another rank's buffer as (rank << 24) | row.
constexpr int PEER_ROW_BITS = 24;
constexpr int PEER_ROW_MASK = (1 << PEER_ROW_BITS) - 1;
constexpr int PEER_MAX_RANKS = 128;

__host__ __device__ inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

template <typename T>
struct TypeInfo;
template <>
struct TypeInfo<float> {
    static constexpr int code = XMA_F32;
    static constexpr int vec = 4;  // elements per 128-bit access
};
template <>
struct TypeInfo<__half> {
    static constexpr int code = XMA_F16;
    static constexpr int vec = 8;
};
template <>
struct TypeInfo<__nv_bfloat16> {
    static constexpr int code = XMA_BF16;
    static constexpr int vec = 8;
};

__device__ __forceinline__ float to_f32(float x) { return x; }
__device__ __forceinline__ float to_f32(__half x) { return __half2float(x); }
__device__ __forceinline__ float to_f32(__nv_bfloat16 x) { return __bfloat162float(x); }

template <typename T>
__device__ __forceinline__ T from_f32(float x);
template <>
__device__ __forceinline__ float from_f32<float>(float x) {
    return x;
}
template <>
__device__ __forceinline__ __half from_f32<__half>(float x) {
    return __float2half_rn(x);
}
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float x) {
    return __float2bfloat16_rn(x);
}

// A 128-bit packet of T. N = 16 / sizeof(T) elements.
template <typename T>
struct alignas(16) Vec16 {
    static constexpr int N = 16 / sizeof(T);
    T v[N];
};

template <typename T>
__device__ __forceinline__ Vec16<T> load16(const T* p) {
    Vec16<T> r;
    *reinterpret_cast<uint4*>(&r) = *reinterpret_cast<const uint4*>(p);
    return r;
}

// Streaming variant: the data is read once, keep it out of the way of reusable lines.
template <typename T>
__device__ __forceinline__ Vec16<T> load16_stream(const T* p) {
    Vec16<T> r;
    *reinterpret_cast<uint4*>(&r) = __ldcs(reinterpret_cast<const uint4*>(p));
    return r;
}

template <typename T>
__device__ __forceinline__ void store16(T* p, const Vec16<T>& r) {
    *reinterpret_cast<uint4*>(p) = *reinterpret_cast<const uint4*>(&r);
}

template <typename T>
__device__ __forceinline__ void store16_stream(T* p, const Vec16<T>& r) {
    __stcs(reinterpret_cast<uint4*>(p), *reinterpret_cast<const uint4*>(&r));
}

// Whole-packet conversions. 16-bit types convert two elements per instruction (cvt.*x2), which halves the
// conversion and packing work of the elementwise kernels compared with one scalar conversion per element.
__device__ __forceinline__ void vec_to_f32(const Vec16<float>& q, float* f) {
#pragma unroll
    for (int i = 0; i < 4; ++i) f[i] = q.v[i];
}
__device__ __forceinline__ void vec_to_f32(const Vec16<__half>& q, float* f) {
    const __half2* h = reinterpret_cast<const __half2*>(&q);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 t = __half22float2(h[i]);
        f[2 * i] = t.x;
        f[2 * i + 1] = t.y;
    }
}
__device__ __forceinline__ void vec_to_f32(const Vec16<__nv_bfloat16>& q, float* f) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 t = __bfloat1622float2(h[i]);
        f[2 * i] = t.x;
        f[2 * i + 1] = t.y;
    }
}
__device__ __forceinline__ void vec_from_f32(const float* f, Vec16<float>& q) {
#pragma unroll
    for (int i = 0; i < 4; ++i) q.v[i] = f[i];
}
__device__ __forceinline__ void vec_from_f32(const float* f, Vec16<__half>& q) {
    __half2* h = reinterpret_cast<__half2*>(&q);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
}
__device__ __forceinline__ void vec_from_f32(const float* f, Vec16<__nv_bfloat16>& q) {
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&q);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
}

__host__ __device__ inline bool is_aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Exact logistic function in fp32 (the torch path of the reference uses F.silu on fp32 values).
__device__ __forceinline__ float sigmoid_f32(float x) { return 1.0f / (1.0f + expf(-x)); }

inline int num_sms() {
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

}  // namespace xma
