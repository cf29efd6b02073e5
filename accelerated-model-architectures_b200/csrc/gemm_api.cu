// C-ABI entry points of the expert grouped GEMMs. `impl` selects the kernel family:
//   0 = automatic: tcgen05 whenever dtype, widths and alignment allow (CTA pairs when experts average
//       >= 1024 rows, one CTA per tile otherwise), CUDA-core path for everything else
//   1 = CUDA-core path        2 = tcgen05 path, one CTA per tile    3 = tcgen05 path, CTA pairs
//   (2 and 3 return XMA_ERR_UNSUPPORTED if the arguments do not qualify)
#include "gemm_internal.h"

#include <cstdlib>
#include <mutex>

namespace xma {

Tuning& tuning() {
    static Tuning t;
    static std::once_flag once;
    std::call_once(once, [] {
        auto env = [](const char* name, int& field) {
            const char* e = getenv(name);
            if (e && *e) field = atoi(e);
        };
        env("XMA_B200_GU_PREFETCH", t.gu_prefetch);
        env("XMA_B200_TMA_PREFETCH", t.tma_prefetch_dist);
        env("XMA_B200_TMA_PREFETCH_MASK", t.tma_prefetch_mask);
        env("XMA_B200_EPI_WARPS", t.epi_warps);
        env("XMA_B200_PLAIN_PAIRS", t.plain_pairs);
        env("XMA_B200_DW_DYNAMIC", t.dw_dynamic);
        env("XMA_B200_DSWIGLU_STAGED", t.dswiglu_staged);
        env("XMA_B200_ODD_TAIL", t.odd_tail);
    });
    return t;
}

uint32_t tune_word() {
    const Tuning& t = tuning();
    uint32_t w = t.gu_prefetch ? 1u : 0u;
    int d = t.tma_prefetch_dist;
    d = d < 0 ? 0 : (d > 255 ? 255 : d);
    w |= static_cast<uint32_t>(d) << 8;
    w |= static_cast<uint32_t>(t.tma_prefetch_mask & 3) << 16;
    return w;
}

}  // namespace xma

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

namespace xma {

int choose_rows_impl(const RowsGemmArgs& g) {
    if (!rows_gemm_tc_supported(g)) return 1;
    const bool plain = g.epilogue == EPI_PLAIN || g.epilogue == EPI_PLAIN_PEER;
    if (!large_experts(g.tile_cap, g.num_experts)) return 2;
    return (plain && !tuning().plain_pairs) ? 2 : 3;
}

int choose_dw_impl(const DwGemmArgs& g) {
    if (!dw_gemm_tc_supported(g)) return 1;
    return large_experts(g.rows_cap / XMA_ROW_PAD, g.num_experts) ? 3 : 2;
}

}  // namespace xma

extern "C" {

int xma_b200_grouped_gemm_rows_peer(const void* a, int64_t a_row_stride, const void* w, int w_layout, void* out,
                                    int64_t out_row_stride, void* aux, int64_t aux_row_stride,
                                    const int32_t* row_map, void* const* out_peers, int peer_world,
                                    int64_t peer_rows_cap, const int32_t* tile_expert, const int32_t* tile_prefix,
                                    int num_experts, int64_t tile_cap, int64_t kd, int64_t n, int epilogue, int dtype,
                                    int impl, int* device_status, cudaStream_t stream) {
    xma::RowsGemmArgs g;
    if (out_peers && (!row_map || epilogue != xma::EPI_PLAIN)) return XMA_ERR_BAD_SHAPE;
    if (out_peers && (peer_world <= 0 || peer_world > xma::PEER_MAX_RANKS || peer_rows_cap <= 0 ||
                      peer_rows_cap > (int64_t{1} << xma::PEER_ROW_BITS)))
        return XMA_ERR_BAD_SHAPE;
    g.out_peers = out_peers;
    g.peer_world = out_peers ? peer_world : 0;
    g.peer_rows_cap = out_peers ? peer_rows_cap : 0;
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
    switch (xma::choose_rows_impl(g)) {
        case 3: {
            // An expert with an odd number of 128-row tiles costs the pair kernel a whole 256-row tile for its last
            // 128 rows. The pairs can go to the pair kernel and the odd last tiles to the one-CTA kernel behind it
            // (which ends at once when there are none); that second launch reads every odd expert's weights once
            // more for 128 rows, so it pays only with few, large experts. Measured on B200, whole layer, switch
            // on against off: 8 experts of about 4100 rows -1.3 % (28.7 against 29.1 ms), 128 experts of about
            // 1024 rows no difference, 64 experts with a Zipf load +2.5 %. Hence: up to 16 experts (switch 1);
            // switch 2 splits for any number of experts.
            const int split = xma::tuning().odd_tail;
            if (out_peers || split == 0 || (split == 1 && g.num_experts > 16)) return xma::rows_gemm_tc2(g);
            g.tune_extra = xma::tc::TUNE_WHOLE_PAIRS_ONLY;
            rc = xma::rows_gemm_tc2(g);
            if (rc) return rc;
            g.tune_extra = xma::tc::TUNE_ODD_LAST_TILE_ONLY;
            return xma::rows_gemm_tc(g);
        }
        case 2: return xma::rows_gemm_tc(g);
        default: return xma::rows_gemm_simt(g);
    }
}

int xma_b200_grouped_gemm_rows(const void* a, int64_t a_row_stride, const void* w, int w_layout, void* out,
                               int64_t out_row_stride, void* aux, int64_t aux_row_stride, const int32_t* row_map,
                               const int32_t* tile_expert, const int32_t* tile_prefix, int num_experts,
                               int64_t tile_cap, int64_t kd, int64_t n, int epilogue, int dtype, int impl,
                               int* device_status, cudaStream_t stream) {
    return xma_b200_grouped_gemm_rows_peer(a, a_row_stride, w, w_layout, out, out_row_stride, aux, aux_row_stride,
                                           row_map, nullptr, 0, 0, tile_expert, tile_prefix, num_experts, tile_cap, kd,
                                           n, epilogue, dtype, impl, device_status, stream);
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
    switch (xma::choose_dw_impl(g)) {
        case 3: return xma::dw_gemm_tc2(g);
        case 2: return xma::dw_gemm_tc(g);
        default: return xma::dw_gemm_simt(g);
    }
}

// The kernel family the automatic choice takes for a problem of this shape on the current device
// (1 CUDA cores, 2 tcgen05 one CTA per tile, 3 tcgen05 CTA pairs); `kind` 0 = rows GEMM, 1 = weight gradient.
// Pointer alignment is assumed (16 bytes), as torch allocations have it.
int xma_b200_grouped_gemm_choice(int kind, int dtype, int num_experts, int64_t tile_cap, int64_t kd, int64_t n,
                                 int w_layout, int epilogue, int peer) {
    static const char aligned[16] __attribute__((aligned(16))) = {0};
    if (kind == 0) {
        xma::RowsGemmArgs g = {};
        g.a = g.w = aligned;
        g.out = g.aux = const_cast<char*>(aligned);
        g.a_stride = kd;
        g.out_stride = (epilogue == xma::EPI_DSWIGLU || epilogue == xma::EPI_DSWIGLU_PACKED) ? 2 * n : n;
        g.aux_stride = (epilogue == xma::EPI_SWIGLU || epilogue == xma::EPI_SWIGLU_PACKED) ? n : 2 * n;
        if (epilogue == xma::EPI_PLAIN) g.aux = nullptr;
        g.w_layout = w_layout;
        g.num_experts = num_experts;
        g.tile_cap = tile_cap;
        g.kd = kd;
        g.n = n;
        g.epilogue = epilogue;
        g.dtype = dtype;
        if (peer) {
            g.epilogue = xma::EPI_PLAIN_PEER;
            g.row_map = reinterpret_cast<const int*>(aligned);
            g.out_peers = reinterpret_cast<void* const*>(aligned);
            g.peer_world = 1;
            g.peer_rows_cap = 1;
        }
        return xma::choose_rows_impl(g);
    }
    xma::DwGemmArgs d = {};
    d.x = d.y = aligned;
    d.dw = const_cast<char*>(aligned);
    d.x_stride = kd;
    d.y_stride = n;
    d.rows_cap = tile_cap * XMA_ROW_PAD;
    d.num_experts = num_experts;
    d.m = kd;
    d.n = n;
    d.dtype = dtype;
    return xma::choose_dw_impl(d);
}

// Tuning switches of the tensor-core kernels (process-wide). key: 0 = gate|up L2 prefetch in the SwiGLU-backward
// epilogue (0/1), 1 = TMA L2 prefetch distance in reduction blocks (0..255), 2 = operands it covers (bit 0 A,
// bit 1 B), 3 = epilogue warps (0 = per-kernel default, 4, 8), 4 = CTA pairs for plain epilogues in the
// automatic choice (0/1), 5 = weight-gradient tiles by atomic ticket, heaviest experts first (0/1). Returns the previous value, or XMA_ERR_BAD_SHAPE for an unknown key. Not synchronised
// with launches in flight on other threads.
int xma_b200_tuning_set(int key, int value) {
    xma::Tuning& t = xma::tuning();
    int* field = nullptr;
    switch (key) {
        case 0: field = &t.gu_prefetch; break;
        case 1: field = &t.tma_prefetch_dist; break;
        case 2: field = &t.tma_prefetch_mask; break;
        case 3: field = &t.epi_warps; break;
        case 4: field = &t.plain_pairs; break;
        case 5: field = &t.dw_dynamic; break;
        case 6: field = &t.dswiglu_staged; break;
        case 7: field = &t.odd_tail; break;
        default: return XMA_ERR_BAD_SHAPE;
    }
    const int previous = *field;
    *field = value;
    return previous;
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

int xma_b200_abi_version(void) { return 3; }

}  // extern "C"
