// Internal launcher interface shared by the grouped-GEMM translation units. Not part of the C ABI.
#pragma once

#include "common.cuh"

namespace xma {

// How the per-expert weight is laid out relative to the product out = A * W_e.
//   W_NK : W_e stored [N, Kd] (reduction dimension contiguous) - forward projections,
//          weight tensor [E, out_features, in_features] used as out = A * W_e^T.
//   W_KN : W_e stored [Kd, N] (output dimension contiguous)   - input-gradient products
//          dA = dOut * W_e with the same stored tensor.
enum WeightLayout { W_NK = 0, W_KN = 1 };

// What happens to the fp32 accumulator tile before it is stored.
//   EPI_PLAIN   : out[dst(r), n] = acc
//   EPI_SWIGLU  : N = 2I. aux[r, 0:2I] = acc (gate | up halves, rounded to the storage type),
//                 out[r, 0:I] = up * gate * sigmoid(gate) computed from the rounded halves.
//   EPI_DSWIGLU : N = I.  aux holds gate|up [r, 0:2I]; out[r, 0:I] = d gate, out[r, I:2I] = d up,
//                 where acc is the gradient of the activation output.
//   EPI_SWIGLU_PACKED / EPI_DSWIGLU_PACKED : the same with gate/up interleaved along the columns
//                 (g, u, g, u, ...) in aux and in the weight rows, as swiglu_packed expects.
//   EPI_DSWIGLU_STAGED : internal (CTA-pair kernel): EPI_DSWIGLU with gate|up fetched and d gate|d up stored by TMA
//                    through shared memory, 32 columns at a time
//   EPI_DSWIGLU_PACKED_STAGED : internal (CTA-pair kernel): the same for the interleaved layout (one 32 x 64 box)
//   EPI_SWIGLU_STAGED : internal (CTA-pair kernel): EPI_SWIGLU with gate|up and the activation stored by TMA
//                    through shared memory, 32 columns at a time
//   EPI_PLAIN_PEER : internal (chosen when out_peers is set): plain store of each row into the buffer of
//                 the rank that row_map names.
enum Epilogue {
    EPI_PLAIN = 0, EPI_SWIGLU = 1, EPI_DSWIGLU = 2, EPI_SWIGLU_PACKED = 3, EPI_DSWIGLU_PACKED = 4, EPI_PLAIN_PEER = 5,
    EPI_DSWIGLU_STAGED = 6, EPI_SWIGLU_STAGED = 7, EPI_DSWIGLU_PACKED_STAGED = 8
};

struct RowsGemmArgs {
    const void* a;             // [rows_cap, Kd] grouped (padded) rows
    int64_t a_stride;          // elements between rows of a
    const void* w;             // [E, N, Kd] (W_NK) or [E, Kd, N] (W_KN), dense
    int w_layout;
    void* out;                 // see Epilogue
    int64_t out_stride;
    void* aux;                 // gate|up buffer for the SwiGLU epilogues, else null
    int64_t aux_stride;
    const int* row_map;        // null: out row = grouped row; else out row = row_map[r], rows < 0 skipped
    void* const* out_peers;    // null, or (plain epilogue with a row_map only) a device table of output
                               // bases, one per rank: row_map[r] = (rank << 24) | row, and the row is
                               // stored to out_peers[rank] instead of `out` (peer memory over NVLink)
    int peer_world;            // entries of out_peers; words naming a rank >= peer_world are skipped and flagged
    int64_t peer_rows_cap;     // rows of every rank's buffer; words naming a row >= this are skipped and flagged
    const int* tile_expert;    // [tile_cap]
    const int* tile_prefix;    // [E+1], tile_prefix[E] = tiles in use
    int num_experts;
    int64_t tile_cap;
    int64_t kd;                // reduction length
    int64_t n;                 // output columns produced by the contraction
    int epilogue;
    int dtype;
    int* device_status;
    cudaStream_t stream;
    uint32_t tune_extra = 0;   // per-launch bits OR-ed into the tuning word (TUNE_WHOLE_PAIRS_ONLY, ...)
};

struct DwGemmArgs {
    const void* x;             // [rows_cap, M] grouped rows: dW_e[m, n] = sum_r x[r, m] * y[r, n]
    int64_t x_stride;
    const void* y;             // [rows_cap, N]
    int64_t y_stride;
    const uint32_t* counts;    // [E] rows per expert
    const int* pad_offsets;    // [E+1] first padded row per expert
    int64_t rows_cap;          // allocated rows of x and y
    int num_experts;
    int64_t m;
    int64_t n;
    void* dw;                  // [E, M, N] dense
    int dtype;
    int* device_status;
    cudaStream_t stream;
};

// Process-wide tuning switches of the tensor-core kernels (xma_b200_tuning_set / XMA_B200_* environment
// variables read once). Defaults are the measured best on B200.
struct Tuning {
    int gu_prefetch = 1;        // SwiGLU-backward epilogue: ask for the next tile's gate|up rows in L2
    int tma_prefetch_dist = 0;  // reduction blocks the TMA producer prefetches into L2 ahead of its loads
    int tma_prefetch_mask = 3;  // bit 0: A operand, bit 1: B operand
    int epi_warps = 0;          // 4 or 8 epilogue warps; 0 = per-kernel default
    int plain_pairs = 1;        // automatic choice: CTA pairs also for the plain epilogues of large experts
    int dw_dynamic = 1;         // weight-gradient pair kernel: tiles by atomic ticket, heaviest experts first
    int dswiglu_staged = 3;     // SwiGLU epilogues of the pair kernel (bit 0: backward, bit 1: forward): their
                                // tiles of gate|up, d gate|d up and the activation go through shared memory by
                                // TMA (when the shapes allow) instead of row-per-thread accesses
    int odd_tail = 1;           // automatic choice: the CTA-pair kernel leaves the odd last 128-row tile of an
                                // expert to a second launch of the one-CTA kernel instead of computing a pair
                                // tile whose second half is empty (1: with up to 16 experts, 2: always, 0: never)
};
Tuning& tuning();

namespace tc {
// Per-launch bits (set by the launcher, not by the tuning switches): the automatic choice may split one rows GEMM
// over two launches, the CTA-pair kernel on the whole pairs of 128-row tiles of every expert and the one-CTA kernel
// on the last tile of the experts that have an odd number of them.
constexpr uint32_t TUNE_WHOLE_PAIRS_ONLY = 1u << 21;
constexpr uint32_t TUNE_ODD_LAST_TILE_ONLY = 1u << 22;
}  // namespace tc

uint32_t tune_word();  // the switches the kernels read, packed (see sm100_common.cuh)

// Which kernel family the automatic choice (impl = 0) takes: 1 CUDA cores, 2 tcgen05 one CTA per tile,
// 3 tcgen05 CTA pairs.
int choose_rows_impl(const RowsGemmArgs& a);
int choose_dw_impl(const struct DwGemmArgs& a);

int rows_gemm_simt(const RowsGemmArgs& a);
int dw_gemm_simt(const DwGemmArgs& a);

// tcgen05 / TMEM / TMA path (bf16 and fp16). `*_supported` is a host-side shape/alignment check.
bool rows_gemm_tc_supported(const RowsGemmArgs& a);
bool dw_gemm_tc_supported(const DwGemmArgs& a);
int rows_gemm_tc(const RowsGemmArgs& a);
int dw_gemm_tc(const DwGemmArgs& a);
// Same contract on CTA pairs (tcgen05 cta_group::2, 256 x 256 tiles).
int rows_gemm_tc2(const RowsGemmArgs& a);
int dw_gemm_tc2(const DwGemmArgs& a);

// Elementwise helpers reused by the unfused epilogues (defined in swiglu.cu).
int swiglu_fwd_launch(const void* g, int64_t gs, const void* u, int64_t us, void* y, int64_t ys, int dtype,
                      int64_t rows, int64_t cols, cudaStream_t st);
int swiglu_bwd_launch(const void* g, int64_t gs, const void* u, int64_t us, const void* dy, int64_t dys, void* dg,
                      int64_t dgs, void* du, int64_t dus, int dtype, int64_t rows, int64_t cols, cudaStream_t st);

}  // namespace xma
