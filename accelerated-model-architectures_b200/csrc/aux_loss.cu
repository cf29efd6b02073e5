// Auxiliary load-balancing loss on the router logits that xma.layers.MoE returns (the reference hands them back
// unused, xma/layers/moe/__init__.py:180, and has no such loss: this is the consumer a training loop adds).
// Definition (Switch Transformer, as commonly used with top-k routing):
//   p[t, :] = softmax(logits[t, :]) in fp32,  P_e = mean_t p[t, e],  f_e = (slots routed to e) / tokens,
//   loss = E * sum_e f_e * P_e;      f_e is a count and carries no gradient.
// The kernels here are the two passes over [tokens, E] (HBM/latency-bound, one warp per token like the top-k
// kernel): column sums of the probabilities, and the gradient
//   d logits[t, j] = p[t, j] * (c_j - sum_e c_e p[t, e]),   c_e = d loss * E * f_e / tokens.
// Counts come from the routing kernels (route_topk_softmax + continuous_count).
#include "common.cuh"

namespace xma {

constexpr int AUX_WARPS = 8;

// Row `t` of the logits as fp32 probabilities: lane l holds columns l, l + 32, ... (NV of them).
template <typename T, int NV>
__device__ __forceinline__ void softmax_row(const T* __restrict__ row, int E, int lane, float (&p)[NV]) {
    float mx = -INFINITY;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int e = lane + 32 * i;
        p[i] = (e < E) ? to_f32(row[e]) : -INFINITY;
        mx = fmaxf(mx, p[i]);
    }
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float sum = 0.0f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int e = lane + 32 * i;
        p[i] = (e < E) ? expf(p[i] - mx) : 0.0f;
        sum += p[i];
    }
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    const float inv = 1.0f / sum;
#pragma unroll
    for (int i = 0; i < NV; ++i) p[i] *= inv;
}

// partial[blockIdx.x, e] = sum over the tokens this CTA handled of p[t, e] (fp32; the caller adds the rows up:
// a fixed order, so the result does not depend on the scheduling of atomics)
template <typename T, int NV>
__global__ void __launch_bounds__(AUX_WARPS * 32)
router_prob_sums_kernel(const T* __restrict__ logits, int64_t stride, int64_t tokens, int E,
                        float* __restrict__ partial) {
    __shared__ float s_acc[AUX_WARPS][32 * NV];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float acc[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i) acc[i] = 0.0f;
    for (int64_t t = static_cast<int64_t>(blockIdx.x) * AUX_WARPS + warp; t < tokens;
         t += static_cast<int64_t>(gridDim.x) * AUX_WARPS) {
        float p[NV];
        softmax_row<T, NV>(logits + t * stride, E, lane, p);
#pragma unroll
        for (int i = 0; i < NV; ++i) acc[i] += p[i];
    }
#pragma unroll
    for (int i = 0; i < NV; ++i) s_acc[warp][lane + 32 * i] = acc[i];
    __syncthreads();
    for (int e = threadIdx.x; e < E; e += AUX_WARPS * 32) {
        float s = 0.0f;
#pragma unroll
        for (int w = 0; w < AUX_WARPS; ++w) s += s_acc[w][e];
        partial[static_cast<int64_t>(blockIdx.x) * E + e] = s;
    }
}

template <typename T, int NV>
__global__ void __launch_bounds__(AUX_WARPS * 32)
load_balance_bwd_kernel(const T* __restrict__ logits, int64_t stride, int64_t tokens, int E,
                        const float* __restrict__ coef, T* __restrict__ d_logits) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float c[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int e = lane + 32 * i;
        c[i] = (e < E) ? coef[e] : 0.0f;
    }
    for (int64_t t = static_cast<int64_t>(blockIdx.x) * AUX_WARPS + warp; t < tokens;
         t += static_cast<int64_t>(gridDim.x) * AUX_WARPS) {
        float p[NV];
        softmax_row<T, NV>(logits + t * stride, E, lane, p);
        float dot = 0.0f;
#pragma unroll
        for (int i = 0; i < NV; ++i) dot += c[i] * p[i];
#pragma unroll
        for (int o = 16; o >= 1; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
        T* out = d_logits + t * E;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int e = lane + 32 * i;
            if (e < E) out[e] = from_f32<T>(p[i] * (c[i] - dot));
        }
    }
}

static int aux_grid(int64_t tokens) {
    const int64_t want = ceil_div(tokens, AUX_WARPS);
    const int64_t cap = static_cast<int64_t>(num_sms()) * 4;
    return static_cast<int>(want < 1 ? 1 : (want > cap ? cap : want));
}

#define XMA_AUX_BY_WIDTH(CALL)                 \
    if (E <= 32) { CALL(1); }                  \
    else if (E <= 64) { CALL(2); }             \
    else if (E <= 128) { CALL(4); }            \
    else if (E <= 256) { CALL(8); }            \
    else if (E <= 512) { CALL(16); }           \
    else { CALL(32); }

template <typename T>
static int prob_sums_t(const void* logits, int64_t stride, int64_t tokens, int E, float* partial, int grid,
                       cudaStream_t stream) {
#define XMA_AUX_FWD(NV) \
    router_prob_sums_kernel<T, NV><<<grid, AUX_WARPS * 32, 0, stream>>>(static_cast<const T*>(logits), stride, tokens, E, partial)
    XMA_AUX_BY_WIDTH(XMA_AUX_FWD)
#undef XMA_AUX_FWD
    return static_cast<int>(cudaGetLastError());
}

template <typename T>
static int lb_bwd_t(const void* logits, int64_t stride, int64_t tokens, int E, const float* coef, void* d_logits,
                    cudaStream_t stream) {
    const int grid = aux_grid(tokens);
#define XMA_AUX_BWD(NV)                                                                                             \
    load_balance_bwd_kernel<T, NV><<<grid, AUX_WARPS * 32, 0, stream>>>(static_cast<const T*>(logits), stride, tokens, \
                                                                        E, coef, static_cast<T*>(d_logits))
    XMA_AUX_BY_WIDTH(XMA_AUX_BWD)
#undef XMA_AUX_BWD
    return static_cast<int>(cudaGetLastError());
}

}  // namespace xma

extern "C" {

int xma_b200_router_prob_partial_rows(int64_t tokens) { return xma::aux_grid(tokens); }

int xma_b200_router_prob_sums(const void* logits, int dtype, int64_t logits_row_stride, int64_t tokens,
                              int num_experts, float* partial, int partial_rows, cudaStream_t stream) {
    if (!partial || (tokens > 0 && !logits)) return XMA_ERR_NULL_POINTER;
    if (tokens < 0 || num_experts <= 0 || num_experts > 1024 || partial_rows <= 0 || logits_row_stride < num_experts)
        return XMA_ERR_BAD_SHAPE;
    const int E = num_experts;
    switch (dtype) {
        case XMA_F32: return xma::prob_sums_t<float>(logits, logits_row_stride, tokens, E, partial, partial_rows, stream);
        case XMA_F16: return xma::prob_sums_t<__half>(logits, logits_row_stride, tokens, E, partial, partial_rows, stream);
        case XMA_BF16:
            return xma::prob_sums_t<__nv_bfloat16>(logits, logits_row_stride, tokens, E, partial, partial_rows, stream);
    }
    return XMA_ERR_BAD_DTYPE;
}

int xma_b200_load_balancing_loss_bwd(const void* logits, int dtype, int64_t logits_row_stride, int64_t tokens,
                                     int num_experts, const float* coef, void* d_logits, cudaStream_t stream) {
    if (tokens == 0) return XMA_OK;
    if (!logits || !coef || !d_logits) return XMA_ERR_NULL_POINTER;
    if (tokens < 0 || num_experts <= 0 || num_experts > 1024 || logits_row_stride < num_experts)
        return XMA_ERR_BAD_SHAPE;
    const int E = num_experts;
    switch (dtype) {
        case XMA_F32: return xma::lb_bwd_t<float>(logits, logits_row_stride, tokens, E, coef, d_logits, stream);
        case XMA_F16: return xma::lb_bwd_t<__half>(logits, logits_row_stride, tokens, E, coef, d_logits, stream);
        case XMA_BF16:
            return xma::lb_bwd_t<__nv_bfloat16>(logits, logits_row_stride, tokens, E, coef, d_logits, stream);
    }
    return XMA_ERR_BAD_DTYPE;
}

}  // extern "C"
