// C-ABI entry points of the expert grouped GEMMs. `impl` selects the kernel family:
//   0 = automatic: tcgen05 whenever dtype, widths and alignment allow (CTA pairs for the SwiGLU
//       epilogues and the weight gradients when experts average >= 1024 rows, one CTA per tile
//       otherwise - measured faster that way on B200), CUDA-core path for everything else
//   1 = CUDA-core path        2 = tcgen05 path, one CTA per tile    3 = tcgen05 path, CTA pairs
//   (2 and 3 return XMA_ERR_UNSUPPORTED if the arguments do not qualify)
#include "gemm_internal.h"

namespace {

// Experts average at least 8 row tiles: a 256-row pair tile then wastes little on odd tile counts.
bool large_experts(int64_t tiles_allocated, int num_experts) {
    return (tiles_allocated - num_experts) >= 8 * static_cast<int64_t>(num_experts);
}

int check_rows(const xma::RowsGemmArgs& g) {
    if (!g.a || !g.w || !g.out || !g.tile_expert || !g.tile_prefix) return XMA_ERR_NULL_POINTER;
    if (g.num_experts <= 0 || g.tile_cap < 0 || g.kd <= 0 || g.n <= 0) return XMA_ERR_BAD_SHAPE;
    if (g.dtype != XMA_F32 && g.dtype != XMA_F16 && g.dtype != XMA_BF16) return XMA_ERR_BAD_DTYPE;
    if (g.w_layout != xma::W_NK && g.w_layout != xma::W_KN) return XMA_ERR_BAD_SHAPE;
    if (g.epilogue < xma::EPI_PLAIN || g.epilogue > xma::EPI_DSWIGLU_PACKED) return XMA_ERR_BAD_SHAPE;
    if (g.epilogue != xma::EPI_PLAIN && !g.aux) return XMA_ERR_NULL_POINTER;
    if ((g.epilogue == xma::EPI_SWIGLU || g.epilogue == xma::EPI_SWIGLU_PACKED) && (g.n % 2)) return XMA_ERR_BAD_SHAPE;
    return XMA_OK;
}

}  // namespace

extern "C" {

int xma_b200_grouped_gemm_rows_peer(const void* a, int64_t a_row_stride, const void* w, int w_layout, void* out,
                                    int64_t out_row_stride, void* aux, int64_t aux_row_stride,
                                    const int32_t* row_map, void* const* out_peers, const int32_t* tile_expert,
                                    const int32_t* tile_prefix, int num_experts, int64_t tile_cap, int64_t kd,
                                    int64_t n, int epilogue, int dtype, int impl, int* device_status,
                                    cudaStream_t stream) {
    xma::RowsGemmArgs g;
    if (out_peers && (!row_map || epilogue != xma::EPI_PLAIN)) return XMA_ERR_BAD_SHAPE;
    g.out_peers = out_peers;
    g.a = a;
    g.a_stride = a_row_stride;
    g.w = w;
    g.w_layout = w_layout;
    g.out = out;
    g.out_stride = out_row_stride;
    g.aux = aux;
    g.aux_stride = aux_row_stride;
    g.row_map = row_map;
    g.tile_expert = tile_expert;
    g.tile_prefix = tile_prefix;
    g.num_experts = num_experts;
    g.tile_cap = tile_cap;
    g.kd = kd;
    g.n = n;
    g.epilogue = epilogue;
    g.dtype = dtype;
    g.device_status = device_status;
    g.stream = stream;
    int rc = check_rows(g);
    if (rc) return rc;
    if (out_peers) g.epilogue = xma::EPI_PLAIN_PEER;  // same contraction, rows stored into the ranks' buffers
    if (impl == 1) return xma::rows_gemm_simt(g);
    if (impl == 2) return xma::rows_gemm_tc(g);
    if (impl == 3) return xma::rows_gemm_tc2(g);
    if (impl != 0) return XMA_ERR_BAD_SHAPE;
    if (xma::rows_gemm_tc_supported(g)) {
        const bool plain = g.epilogue == xma::EPI_PLAIN || g.epilogue == xma::EPI_PLAIN_PEER;
        if (!plain && large_experts(g.tile_cap, g.num_experts)) return xma::rows_gemm_tc2(g);
        return xma::rows_gemm_tc(g);
    }
    return xma::rows_gemm_simt(g);
}

int xma_b200_grouped_gemm_rows(const void* a, int64_t a_row_stride, const void* w, int w_layout, void* out,
                               int64_t out_row_stride, void* aux, int64_t aux_row_stride, const int32_t* row_map,
                               const int32_t* tile_expert, const int32_t* tile_prefix, int num_experts,
                               int64_t tile_cap, int64_t kd, int64_t n, int epilogue, int dtype, int impl,
                               int* device_status, cudaStream_t stream) {
    return xma_b200_grouped_gemm_rows_peer(a, a_row_stride, w, w_layout, out, out_row_stride, aux, aux_row_stride,
                                           row_map, nullptr, tile_expert, tile_prefix, num_experts, tile_cap, kd, n,
                                           epilogue, dtype, impl, device_status, stream);
}

int xma_b200_grouped_gemm_dw(const void* x, int64_t x_row_stride, const void* y, int64_t y_row_stride,
                             const uint32_t* counts, const int32_t* pad_offsets, int64_t rows_cap, int num_experts,
                             int64_t m, int64_t n, void* dw, int dtype, int impl, int* device_status,
                             cudaStream_t stream) {
    if (!x || !y || !counts || !pad_offsets || !dw) return XMA_ERR_NULL_POINTER;
    if (num_experts <= 0 || m <= 0 || n <= 0 || rows_cap < 0) return XMA_ERR_BAD_SHAPE;
    if (dtype != XMA_F32 && dtype != XMA_F16 && dtype != XMA_BF16) return XMA_ERR_BAD_DTYPE;
    xma::DwGemmArgs g;
    g.x = x;
    g.x_stride = x_row_stride;
    g.y = y;
    g.y_stride = y_row_stride;
    g.counts = counts;
    g.pad_offsets = pad_offsets;
    g.rows_cap = rows_cap;
    g.num_experts = num_experts;
    g.m = m;
    g.n = n;
    g.dw = dw;
    g.dtype = dtype;
    g.device_status = device_status;
    g.stream = stream;
    if (impl == 1) return xma::dw_gemm_simt(g);
    if (impl == 2) return xma::dw_gemm_tc(g);
    if (impl == 3) return xma::dw_gemm_tc2(g);
    if (impl != 0) return XMA_ERR_BAD_SHAPE;
    if (xma::dw_gemm_tc_supported(g)) {
        if (large_experts(rows_cap / XMA_ROW_PAD, num_experts)) return xma::dw_gemm_tc2(g);
        return xma::dw_gemm_tc(g);
    }
    return xma::dw_gemm_simt(g);
}

// 1 when the automatic choice for these arguments is the tcgen05 path.
int xma_b200_grouped_gemm_uses_tensor_cores(int dtype, int64_t kd, int64_t n) {
    return ((dtype == XMA_BF16 || dtype == XMA_F16) && kd % 8 == 0 && n % 8 == 0) ? 1 : 0;
}

const char* xma_b200_error_string(int code) {
    switch (code) {
        case XMA_OK: return "ok";
        case XMA_ERR_NULL_POINTER: return "null pointer argument";
        case XMA_ERR_BAD_DTYPE: return "unsupported dtype code";
        case XMA_ERR_BAD_SHAPE: return "invalid shape, size or flag argument";
        case XMA_ERR_SCRATCH_TOO_SMALL: return "scratch buffer too small";
        case XMA_ERR_UNSUPPORTED: return "arguments not supported by the requested kernel";
        case XMA_ERR_MISALIGNED: return "pointer, stride or width violates the alignment rule";
        case XMA_ERR_TENSOR_MAP: return "TMA tensor map creation failed";
        case XMA_ERR_TOO_LARGE: return "problem size exceeds the supported range";
    }
    if (code > 0) return cudaGetErrorString(static_cast<cudaError_t>(code));
    return "unknown error";
}

int xma_b200_abi_version(void) { return 1; }

}  // extern "C"
