// pack_sequence / unpack_sequence (xma/functional/sequence_packing/__init__.py:39-132; semantics as in
// torch_implementation.py:9-48; kernels replaced: cuda_implementation.py:17-98 and triton_implementation.py).
//   padded  [B, S, row]  : B sequences, each padded on the left or on the right to S tokens
//   packed  [T, row]     : the valid tokens of sequence 0, then of sequence 1, ... (T = cu_seqlens[B])
//   cu_seqlens [B + 1]   : cumulative sequence lengths, cu_seqlens[0] = 0
// Both layouts keep a token's `row` elements contiguous and a sequence's tokens consecutive, so sequence b is ONE
// contiguous byte range in either layout:
//   packed : [cu[b] * row_bytes, cu[b + 1] * row_bytes)
//   padded : [(b * S + pad_b) * row_bytes, ... + len_b * row_bytes),  pad_b = S - len_b (left) or 0 (right)
// and packing is B segment copies. The kernels therefore work on bytes, not on elements and dtypes: the copy
// unit is the largest power of two (16 bytes at most) that divides row_bytes and both base addresses, which keeps
// every segment boundary on a unit boundary. HBM-bound: 2 bytes moved per byte of valid tokens (pack), and for
// unpack the zero padding is written by the same kernel (the reference zero-fills the whole output first,
// cuda_implementation.py:182, and then writes the tokens over it: one more pass over the output).
// A CTA takes CHUNK units of one sequence's padded range (blockIdx.x -> (sequence, chunk)); the units of a thread
// are all loaded before the first is stored.
#include "common.cuh"

namespace xma {

constexpr int SP_THREADS = 256;
constexpr int SP_UNROLL = 4;
constexpr int SP_CHUNK = SP_THREADS * SP_UNROLL;  // units per CTA

template <typename CuT>
__device__ __forceinline__ bool sequence_range(const CuT* __restrict__ cu, int64_t b, int64_t seq_len,
                                               int64_t total_tokens, int left, int64_t& start, int64_t& len,
                                               int64_t& pad) {
    const int64_t s = static_cast<int64_t>(cu[b]), e = static_cast<int64_t>(cu[b + 1]);
    start = s;
    len = e - s;
    pad = left ? seq_len - len : 0;
    // a sequence longer than the padded length, or one that leaves the packed buffer, is skipped as a whole
    return s >= 0 && e >= s && e <= total_tokens && len <= seq_len;
}

// PACK = true : padded -> packed; zeros in packed rows behind the last sequence
// PACK = false: packed -> padded, zeros in the padding
template <typename U, typename CuT, bool PACK>
__global__ void __launch_bounds__(SP_THREADS)
sequence_packing_kernel(const U* __restrict__ src, U* __restrict__ dst, const CuT* __restrict__ cu, int64_t batch,
                        int64_t seq_len, int64_t total_tokens, int64_t row_units, int left, unsigned chunks_per_sequence,
                        int* __restrict__ status) {
    const int64_t b = blockIdx.x / chunks_per_sequence;
    const int64_t chunk = blockIdx.x - b * chunks_per_sequence;
    int64_t start, len, pad;
    const bool ok = sequence_range(cu, b, seq_len, total_tokens, left, start, len, pad);
    if (!ok) {
        if (status && threadIdx.x == 0 && chunk == 0) atomicOr(status, XMA_DEV_ID_OUT_OF_RANGE);
        len = 0;
        pad = left ? seq_len : 0;
    }
    const int64_t valid_lo = pad * row_units, valid_hi = (pad + len) * row_units;  // within the padded sequence
    const int64_t padded_base = b * seq_len * row_units;
    const int64_t packed_base = start * row_units - valid_lo;  // + position in the padded sequence = packed unit
    const int64_t lo = chunk * SP_CHUNK;
    const int64_t limit = seq_len * row_units;
    if (PACK && b == batch - 1) {
        // rows of the packed buffer behind the last sequence (total_tokens > cu_seqlens[batch]; normally none):
        // zeros, shared out among the CTAs of the last sequence
        const int64_t last = static_cast<int64_t>(cu[batch]);
        if (last >= 0 && last < total_tokens)
            for (int64_t p = last * row_units + chunk * SP_THREADS + threadIdx.x; p < total_tokens * row_units;
                 p += static_cast<int64_t>(chunks_per_sequence) * SP_THREADS)
                dst[p] = U{};
    }
    if (PACK && (lo >= valid_hi || lo + SP_CHUNK <= valid_lo)) return;  // this chunk is padding only

    U v[SP_UNROLL];
#pragma unroll
    for (int k = 0; k < SP_UNROLL; ++k) {
        const int64_t p = lo + threadIdx.x + static_cast<int64_t>(k) * SP_THREADS;
        const bool valid = p >= valid_lo && p < valid_hi;
        if (PACK) {
            if (valid) v[k] = __ldcs(src + padded_base + p);
        } else {
            v[k] = U{};
            if (valid) v[k] = __ldcs(src + packed_base + p);
        }
    }
#pragma unroll
    for (int k = 0; k < SP_UNROLL; ++k) {
        const int64_t p = lo + threadIdx.x + static_cast<int64_t>(k) * SP_THREADS;
        const bool valid = p >= valid_lo && p < valid_hi;
        if (PACK) {
            if (valid) __stcs(dst + packed_base + p, v[k]);
        } else {
            if (p < limit) __stcs(dst + padded_base + p, v[k]);
        }
    }
}

template <typename U, typename CuT>
static int launch_sequence_packing(const void* src, void* dst, const void* cu, int64_t batch, int64_t seq_len,
                                   int64_t total_tokens, int64_t row_bytes, int left, bool pack, int* status,
                                   cudaStream_t stream) {
    const int64_t row_units = row_bytes / static_cast<int64_t>(sizeof(U));
    const int64_t chunks = ceil_div(seq_len * row_units, static_cast<int64_t>(SP_CHUNK));
    if (chunks > 0x7fffffffll || batch * chunks > 0x7fffffffll) return XMA_ERR_TOO_LARGE;
    const unsigned grid = static_cast<unsigned>(batch * chunks);
    if (pack)
        sequence_packing_kernel<U, CuT, true><<<grid, SP_THREADS, 0, stream>>>(
            static_cast<const U*>(src), static_cast<U*>(dst), static_cast<const CuT*>(cu), batch, seq_len, total_tokens,
            row_units, left, static_cast<unsigned>(chunks), status);
    else
        sequence_packing_kernel<U, CuT, false><<<grid, SP_THREADS, 0, stream>>>(
            static_cast<const U*>(src), static_cast<U*>(dst), static_cast<const CuT*>(cu), batch, seq_len, total_tokens,
            row_units, left, static_cast<unsigned>(chunks), status);
    return static_cast<int>(cudaGetLastError());
}

template <typename U>
static int sequence_packing_by_index_type(const void* src, void* dst, const void* cu, int cu_dtype, int64_t batch,
                                          int64_t seq_len, int64_t total_tokens, int64_t row_bytes, int left,
                                          bool pack, int* status, cudaStream_t stream) {
    // uint32 offsets (what the reference's tests pass) take the int32 code: values below 2^31 read the same
    if (cu_dtype == XMA_I32)
        return launch_sequence_packing<U, int32_t>(src, dst, cu, batch, seq_len, total_tokens, row_bytes, left, pack,
                                                   status, stream);
    if (cu_dtype == XMA_I64)
        return launch_sequence_packing<U, int64_t>(src, dst, cu, batch, seq_len, total_tokens, row_bytes, left, pack,
                                                   status, stream);
    return XMA_ERR_BAD_DTYPE;
}

static int sequence_packing(const void* src, void* dst, const void* cu, int cu_dtype, int64_t batch, int64_t seq_len,
                            int64_t total_tokens, int64_t row_bytes, int left, bool pack, int* status,
                            cudaStream_t stream) {
    if (batch < 0 || seq_len < 0 || total_tokens < 0 || row_bytes < 0) return XMA_ERR_BAD_SHAPE;
    if (batch == 0 || seq_len == 0 || row_bytes == 0) return XMA_OK;
    if (pack && total_tokens == 0) return XMA_OK;  // nothing to write
    if (!cu || !dst || (!src && total_tokens > 0)) return XMA_ERR_NULL_POINTER;
    const uintptr_t bits = reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst) |
                           static_cast<uintptr_t>(row_bytes);
#define XMA_SP_CALL(U) \
    sequence_packing_by_index_type<U>(src, dst, cu, cu_dtype, batch, seq_len, total_tokens, row_bytes, left, pack, status, stream)
    if ((bits & 15u) == 0) return XMA_SP_CALL(uint4);
    if ((bits & 7u) == 0) return XMA_SP_CALL(uint2);
    if ((bits & 3u) == 0) return XMA_SP_CALL(uint32_t);
    if ((bits & 1u) == 0) return XMA_SP_CALL(uint16_t);
    return XMA_SP_CALL(uint8_t);
#undef XMA_SP_CALL
}

}  // namespace xma

extern "C" {

int xma_b200_pack_sequence(const void* padded, void* packed, const void* cu_seqlens, int cu_dtype, int64_t batch,
                           int64_t seq_len, int64_t total_tokens, int64_t row_bytes, int left_padding,
                           int* device_status, cudaStream_t stream) {
    return xma::sequence_packing(padded, packed, cu_seqlens, cu_dtype, batch, seq_len, total_tokens, row_bytes,
                                 left_padding, true, device_status, stream);
}

int xma_b200_unpack_sequence(const void* packed, void* padded, const void* cu_seqlens, int cu_dtype, int64_t batch,
                             int64_t seq_len, int64_t total_tokens, int64_t row_bytes, int left_padding,
                             int* device_status, cudaStream_t stream) {
    return xma::sequence_packing(packed, padded, cu_seqlens, cu_dtype, batch, seq_len, total_tokens, row_bytes,
                                 left_padding, false, device_status, stream);
}

}  // extern "C"
