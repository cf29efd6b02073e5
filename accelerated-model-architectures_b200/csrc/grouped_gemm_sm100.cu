// Expert grouped GEMMs on the Blackwell tensor cores (sm_100a): tcgen05.mma with fp32
// accumulators in tensor memory, operands staged in shared memory by TMA (128-byte swizzle), a
// persistent per-expert tile scheduler, and the SwiGLU forward/backward fused into the epilogue.
//
// Replaces scatter2scatter (xma/layers/moe/triton_implementation/scatter_kernel.py:54-183) and
// group_bwd_W (xma/layers/moe/triton_implementation/group_backward_kernel.py:13-128). The row
// gather/scatter those kernels do with pointer arithmetic is split off: inputs arrive in the padded
// grouped layout (rows of an expert contiguous, padded to 128), outputs either stay grouped or are
// scattered through `row_map` by the epilogue.
//
// One CTA per SM, 192 or 320 threads:
//   warp 0      : TMA producer (one lane)            -> full[stage]
//   warp 1      : tensor-memory allocation, MMA issue (one lane) -> empty[stage], acc_full[buf]
//   warps 2..   : epilogue (4 or 8 warps); warp w reads the 32-lane quarter (w & 3) of tensor memory
//                 and, with 8 warps, half of the tile's columns -> acc_empty[buf]
// The accumulator is double buffered (2 x 256 columns), so the epilogue of a tile overlaps the
// main loop of the next one. Every wait is bounded: on expiry the CTA raises a flag, sets the
// wait-timeout bit of the device status word, leaves its loops and still frees its tensor memory.
#include "sm100_common.cuh"

namespace xma {
namespace tc {

struct Shared {
    uint8_t* stage_base;  // 1024-byte aligned
    int* tile_prefix;     // [E + 1]
    int* odd_prefix;      // [E + 1] experts with an odd number of row tiles in front of each expert (rows GEMM,
                          // odd-last-tile launches only)
    uint64_t* full;       // [STAGES]
    uint64_t* empty;      // [STAGES]
    uint64_t* acc_full;   // [2]
    uint64_t* acc_empty;  // [2]
    uint32_t* tmem_ptr;
    volatile int* abort_flag;
    uint8_t* peer_stage;  // [PEER_STAGE_BYTES], 16-byte aligned
};

__device__ __forceinline__ Shared carve_smem(uint8_t* raw) {
    Shared s;
    const uint32_t a = smem_u32(raw);
    uint8_t* base = raw + ((1024u - (a & 1023u)) & 1023u);
    s.stage_base = base;
    uint8_t* p = base + static_cast<size_t>(STAGES) * STAGE_BYTES;
    s.tile_prefix = reinterpret_cast<int*>(p);
    p += (MAX_EXPERTS + 1) * sizeof(int);
    s.odd_prefix = reinterpret_cast<int*>(p);
    p += (MAX_EXPERTS + 1) * sizeof(int);
    p = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(p) + 7) & ~static_cast<uintptr_t>(7));
    s.full = reinterpret_cast<uint64_t*>(p);
    s.empty = s.full + STAGES;
    s.acc_full = s.empty + STAGES;
    s.acc_empty = s.acc_full + 2;
    s.tmem_ptr = reinterpret_cast<uint32_t*>(s.acc_empty + 2);
    s.abort_flag = reinterpret_cast<volatile int*>(s.tmem_ptr + 1);
    s.peer_stage = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(s.tmem_ptr + 2) + 15) & ~static_cast<uintptr_t>(15));
    return s;
}

// Common prologue: barriers, tensor-memory allocation. Returns the tensor-memory base address.
__device__ __forceinline__ uint32_t prologue(const Shared& s, int warp, int lane) {
    if (threadIdx.x == 0) {
        for (int i = 0; i < STAGES; ++i) {
            mbar_init(&s.full[i], 1);
            mbar_init(&s.empty[i], 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&s.acc_full[i], 1);
            mbar_init(&s.acc_empty[i], blockDim.x - 64);
        }
        *s.abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(s.tmem_ptr, TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    (void)lane;
    return *s.tmem_ptr;
}

__device__ __forceinline__ void teardown(const Shared& s, uint32_t tmem_base, int warp, int* status) {
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
    if (threadIdx.x == 0 && *s.abort_flag && status) atomicOr(status, XMA_DEV_WAIT_TIMEOUT);
}

// One pipeline stage of MMA issue: four tcgen05.mma over the 64-element reduction block.
template <bool A_MN, bool B_MN>
__device__ __forceinline__ void issue_stage(uint32_t a_saddr, uint32_t b_saddr, uint32_t tmem_d, uint32_t idesc,
                                            bool first_block) {
    const uint64_t da = smem_desc(a_saddr, A_MN);
    const uint64_t db = smem_desc(b_saddr, B_MN);
#pragma unroll
    for (int k = 0; k < BK / UMMA_K; ++k) {
        umma_f16(tmem_d, da + static_cast<uint64_t>(k * desc_k_step(A_MN)),
                 db + static_cast<uint64_t>(k * desc_k_step(B_MN)), idesc, (first_block && k == 0) ? 0u : 1u);
    }
}

// ======================================================================================================
// Rows GEMM: out[dst(r), :] = epilogue( A[r, :] * W_e ), r over the padded grouped rows.
// Work order: expert-major; inside an expert groups of ROWS_RASTER_GROUP row tiles x all column tiles
// (raster_tile), so the CTAs of one wave share both a few row blocks and a few weight tiles.
// ======================================================================================================
constexpr int ROWS_RASTER_GROUP = 16;  // 148 CTAs: about 16 row tiles x 9 column tiles per wave

struct RowsWork {
    int m_tile, n_tile, e;
};

// `tile_prefix` may be a slice of a longer table (experts [a, b) of a layer: the expert-parallel layer runs its
// experts group by group), so its first entry is not necessarily 0: work items count from tile_prefix[0].
__device__ __forceinline__ RowsWork decode_rows(const int* tile_prefix, int E, int n_tiles, int64_t w) {
    const int base = tile_prefix[0];
    // largest e with (tile_prefix[e] - base) * n_tiles <= w
    int lo = 0, hi = E;  // invariant: (prefix[lo] - base) * n_tiles <= w < (prefix[hi] - base) * n_tiles
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (static_cast<int64_t>(tile_prefix[mid] - base) * n_tiles <= w) lo = mid;
        else hi = mid;
    }
    RowsWork r;
    r.e = lo;
    const int64_t local = w - static_cast<int64_t>(tile_prefix[lo] - base) * n_tiles;
    const int mt = tile_prefix[lo + 1] - tile_prefix[lo];
    int m;
    raster_tile(local, mt, n_tiles, ROWS_RASTER_GROUP, m, r.n_tile);
    r.m_tile = tile_prefix[lo] + m;
    return r;
}

// The work items of a launch that takes only the last row tile of every expert with an odd number of them (the
// whole pairs of tiles went to the CTA-pair kernel): expert-major, all column tiles of that one row tile.
__device__ __forceinline__ RowsWork decode_odd_rows(const int* tile_prefix, const int* odd_prefix, int E, int n_tiles,
                                                    int64_t w) {
    int lo = 0, hi = E;  // invariant: odd_prefix[lo] * n_tiles <= w < odd_prefix[hi] * n_tiles
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (static_cast<int64_t>(odd_prefix[mid]) * n_tiles <= w) lo = mid;
        else hi = mid;
    }
    RowsWork r;
    r.e = lo;
    r.n_tile = static_cast<int>(w - static_cast<int64_t>(odd_prefix[lo]) * n_tiles);
    r.m_tile = tile_prefix[lo + 1] - 1;
    return r;
}

template <typename T, int WL, int EPI>
__global__ void __launch_bounds__(THREADS, 1)
rows_gemm_tc_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                    T* __restrict__ out, int64_t out_stride, T* __restrict__ aux, int64_t aux_stride,
                    const int* __restrict__ row_map, void* const* __restrict__ out_peers, int peer_world,
                    int64_t peer_rows_cap, const int* __restrict__ g_tile_prefix, int E, int kd, int n,
                    uint32_t idesc, uint32_t tune, int* __restrict__ status) {
    extern __shared__ __align__(16) uint8_t smem_raw[];
    const Shared s = carve_smem(smem_raw);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    for (int i = threadIdx.x; i <= E; i += blockDim.x) s.tile_prefix[i] = g_tile_prefix[i];
    const bool odd_only = (tune & TUNE_ODD_LAST_TILE_ONLY) != 0;
    if (odd_only) {
        __syncthreads();
        if (threadIdx.x == 32) {
            int run = 0;
            for (int e = 0; e < E; ++e) {
                s.odd_prefix[e] = run;
                run += (s.tile_prefix[e + 1] - s.tile_prefix[e]) & 1;
            }
            s.odd_prefix[E] = run;
        }
    }
    const uint32_t tmem_base = prologue(s, warp, lane);

    constexpr bool B_MN = (WL == W_KN);
    const int half_n = n / 2;  // SwiGLU: width of the activation
    const int n_tiles = (EPI == EPI_SWIGLU) ? (half_n + 127) / 128 : (n + BN - 1) / BN;
    const int k_blocks = (kd + BK - 1) / BK;
    const int64_t total =
        static_cast<int64_t>(odd_only ? s.odd_prefix[E] : s.tile_prefix[E] - s.tile_prefix[0]) * n_tiles;
    auto decode = [&](int64_t w) {
        return odd_only ? decode_odd_rows(s.tile_prefix, s.odd_prefix, E, n_tiles, w)
                        : decode_rows(s.tile_prefix, E, n_tiles, w);
    };

    if (warp == 0) {
        if (lane == 0) {
            uint32_t it = 0;
            for (int64_t w = blockIdx.x; w < total; w += gridDim.x) {
                const RowsWork wk = decode(w);
                bool ok = true;
                for (int kb = 0; kb < k_blocks && ok; ++kb, ++it) {
                    const int st = it % STAGES;
                    ok = mbar_wait(&s.empty[st], ((it / STAGES) & 1u) ^ 1u, s.abort_flag);
                    if (!ok) break;
                    uint8_t* sa = s.stage_base + static_cast<size_t>(st) * STAGE_BYTES;
                    uint8_t* sb = sa + A_STAGE_BYTES;
                    mbar_expect_tx(&s.full[st], STAGE_BYTES);
                    tma_load_2d(sa, &tm_a, &s.full[st], kb * BK, wk.m_tile * BM);
                    if (!B_MN) {
                        // weight stored [E * n, kd]: two boxes of 128 rows x 64 reduction elements
                        int r0, r1;
                        if (EPI == EPI_SWIGLU) {
                            r0 = wk.e * n + wk.n_tile * 128;  // gate rows
                            r1 = r0 + half_n;                 // matching up rows
                        } else {
                            r0 = wk.e * n + wk.n_tile * BN;
                            r1 = r0 + 128;
                        }
                        tma_load_2d(sb, &tm_b, &s.full[st], kb * BK, r0);
                        tma_load_2d(sb + 128 * BK * 2, &tm_b, &s.full[st], kb * BK, r1);
                    } else {
                        // weight stored [E * kd, n]: four boxes of 64 columns x 64 reduction rows
#pragma unroll
                        for (int j = 0; j < BN / 64; ++j)
                            tma_load_2d(sb + j * CHUNK_BYTES, &tm_b, &s.full[st], wk.n_tile * BN + j * 64,
                                        wk.e * kd + kb * BK);
                    }
                }
                if (!ok) break;
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            uint32_t it = 0, lt = 0;
            for (int64_t w = blockIdx.x; w < total; w += gridDim.x, ++lt) {
                const uint32_t buf = lt & 1u;
                if (!mbar_wait(&s.acc_empty[buf], ((lt >> 1) & 1u) ^ 1u, s.abort_flag)) break;
                tc_fence_after();
                const uint32_t tmem_d = tmem_base + buf * BN;
                bool ok = true;
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const int st = it % STAGES;
                    ok = mbar_wait(&s.full[st], (it / STAGES) & 1u, s.abort_flag);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t sa = smem_u32(s.stage_base + static_cast<size_t>(st) * STAGE_BYTES);
                    issue_stage<false, B_MN>(sa, sa + A_STAGE_BYTES, tmem_d, idesc, kb == 0);
                    umma_commit(&s.empty[st]);
                }
                if (!ok) break;
                umma_commit(&s.acc_full[buf]);
            }
        }
    } else {
        const int quarter = warp & 3;          // tensor-memory lanes [32 * quarter, 32 * quarter + 32)
        const int parts = (static_cast<int>(blockDim.x) - 64) >> 7;  // warps per lane quarter: 1 or 2
        const int part = (warp - 2) >> 2;                            // which share of the columns this warp stores
        const int chunks = (BN / 32) / parts;                        // 32-column chunks per warp
        const int row_in_tile = quarter * 32 + lane;
        // one staging region per epilogue warp when there are four of them
        uint8_t* peer_stage = (parts == 1) ? s.peer_stage + (warp - 2) * PEER_STAGE_WARP_BYTES : nullptr;
        uint32_t lt = 0;
        for (int64_t w = blockIdx.x; w < total; w += gridDim.x, ++lt) {
            const RowsWork wk = decode(w);
            const uint32_t buf = lt & 1u;
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + buf * BN;
            const int64_t r = static_cast<int64_t>(wk.m_tile) * BM + row_in_tile;
            if ((EPI == EPI_DSWIGLU || EPI == EPI_DSWIGLU_PACKED) && (tune & TUNE_GU_PREFETCH) &&
                w + gridDim.x < total) {
                const RowsWork nx = decode(w + gridDim.x);
                prefetch_gate_up<T, EPI>(aux, aux_stride, static_cast<int64_t>(nx.m_tile) * BM + row_in_tile,
                                         nx.n_tile, n, part, chunks);
            }
            if (!rows_epilogue_tile<T, EPI>(&s.acc_full[buf], (lt >> 1) & 1u, s.abort_flag, taddr, r, true, wk.n_tile, n,
                                            half_n, out, out_stride, aux, aux_stride, row_map, out_peers, peer_world,
                                            peer_rows_cap, status, peer_stage, part, chunks))
                break;
            tc_fence_before();
            mbar_arrive(&s.acc_empty[buf]);
        }
    }
    teardown(s, tmem_base, warp, status);
}

// ======================================================================================================
// Weight-gradient GEMM: dW_e[m, n] = sum over the rows r of expert e of X[r, m] * Y[r, n].
// Both operands are MN-major (the reduction runs over rows). Experts without rows get zeros.
// Work order: expert-major, then groups of 8 row tiles x all column tiles (row tile fastest).
// ======================================================================================================
template <typename T>
__global__ void __launch_bounds__(THREADS, 1)
dw_gemm_tc_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_y,
                  const uint32_t* __restrict__ counts, const int* __restrict__ pad_offsets, int E, int m, int n,
                  T* __restrict__ dw, uint32_t idesc, int* __restrict__ status) {
    extern __shared__ __align__(16) uint8_t smem_raw[];
    const Shared s = carve_smem(smem_raw);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t tmem_base = prologue(s, warp, lane);

    const int m_tiles = (m + BM - 1) / BM;
    const int n_tiles = (n + BN - 1) / BN;
    const int64_t total = static_cast<int64_t>(E) * m_tiles * n_tiles;

    if (warp == 0) {
        if (lane == 0) {
            uint32_t it = 0;
            for (int64_t w = blockIdx.x; w < total; w += gridDim.x) {
                const DwWork wk = decode_dw(w, m_tiles, n_tiles);
                const int k_blocks = (static_cast<int>(counts[wk.e]) + BK - 1) / BK;
                const int row0 = pad_offsets[wk.e];
                bool ok = true;
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const int st = it % STAGES;
                    ok = mbar_wait(&s.empty[st], ((it / STAGES) & 1u) ^ 1u, s.abort_flag);
                    if (!ok) break;
                    uint8_t* sa = s.stage_base + static_cast<size_t>(st) * STAGE_BYTES;
                    uint8_t* sb = sa + A_STAGE_BYTES;
                    mbar_expect_tx(&s.full[st], STAGE_BYTES);
#pragma unroll
                    for (int j = 0; j < BM / 64; ++j)
                        tma_load_2d(sa + j * CHUNK_BYTES, &tm_x, &s.full[st], wk.m_tile * BM + j * 64,
                                    row0 + kb * BK);
#pragma unroll
                    for (int j = 0; j < BN / 64; ++j)
                        tma_load_2d(sb + j * CHUNK_BYTES, &tm_y, &s.full[st], wk.n_tile * BN + j * 64,
                                    row0 + kb * BK);
                }
                if (!ok) break;
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            uint32_t it = 0, lt = 0;
            for (int64_t w = blockIdx.x; w < total; w += gridDim.x) {
                const DwWork wk = decode_dw(w, m_tiles, n_tiles);
                const int k_blocks = (static_cast<int>(counts[wk.e]) + BK - 1) / BK;
                if (k_blocks == 0) continue;  // the epilogue writes zeros without an accumulator
                const uint32_t buf = lt & 1u;
                if (!mbar_wait(&s.acc_empty[buf], ((lt >> 1) & 1u) ^ 1u, s.abort_flag)) break;
                tc_fence_after();
                const uint32_t tmem_d = tmem_base + buf * BN;
                bool ok = true;
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const int st = it % STAGES;
                    ok = mbar_wait(&s.full[st], (it / STAGES) & 1u, s.abort_flag);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t sa = smem_u32(s.stage_base + static_cast<size_t>(st) * STAGE_BYTES);
                    issue_stage<true, true>(sa, sa + A_STAGE_BYTES, tmem_d, idesc, kb == 0);
                    umma_commit(&s.empty[st]);
                }
                if (!ok) break;
                umma_commit(&s.acc_full[buf]);
                ++lt;
            }
        }
    } else {
        const int quarter = warp & 3;
        const int parts = (static_cast<int>(blockDim.x) - 64) >> 7;
        const int part = (warp - 2) >> 2;
        const int chunks = (BN / 32) / parts;
        const int row_in_tile = quarter * 32 + lane;
        uint32_t lt = 0;
        for (int64_t w = blockIdx.x; w < total; w += gridDim.x) {
            const DwWork wk = decode_dw(w, m_tiles, n_tiles);
            const bool empty_expert = (counts[wk.e] == 0u);
            const int row = wk.m_tile * BM + row_in_tile;
            const int n0 = wk.n_tile * BN;
            T* dst = dw + (static_cast<int64_t>(wk.e) * m + row) * n + n0;
            if (empty_expert) {
                if (row < m) {
                    const uint4 z = make_uint4(0u, 0u, 0u, 0u);
                    for (int c = part * chunks * 32; c < (part + 1) * chunks * 32 && n0 + c < n; c += 8)
                        *reinterpret_cast<uint4*>(dst + c) = z;
                }
                continue;
            }
            const uint32_t buf = lt & 1u;
            if (!mbar_wait_epilogue(&s.acc_full[buf], (lt >> 1) & 1u, s.abort_flag)) break;
            tc_fence_after();
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + buf * BN;
#pragma unroll 1
            for (int c = part * chunks; c < (part + 1) * chunks; ++c) {
                uint32_t v[32];
                tmem_ld32(taddr + c * 32, v);
                tmem_ld_wait();
                const int col = n0 + c * 32;
                if (row < m && col < n) {
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        if (col + 8 * i < n)
                            *reinterpret_cast<uint4*>(dst + c * 32 + 8 * i) =
                                pack8<T>(reinterpret_cast<const float*>(&v[8 * i]));
                    }
                }
            }
            tc_fence_before();
            mbar_arrive(&s.acc_empty[buf]);
            ++lt;
        }
    }
    teardown(s, tmem_base, warp, status);
}

// ---- host side ---------------------------------------------------------------------------------------

template <typename K>
static int set_smem(K kernel) {
    apply_epilogue_tuning();
    return set_dynamic_smem_once(kernel, SMEM_BYTES);
}

template <typename T, int WL, int EPI>
static int launch_rows(const RowsGemmArgs& g, const CUtensorMap& ta, const CUtensorMap& tb) {
    auto kernel = rows_gemm_tc_kernel<T, WL, EPI>;
    int rc = set_smem(kernel);
    if (rc) return rc;
    const uint32_t idesc = make_idesc(g.dtype, false, WL == W_KN);
    // (rows bound for other ranks are staged per epilogue warp: always four warps then)
    const int threads = (EPI == EPI_PLAIN_PEER) ? 64 + 32 * 4 : block_threads((EPI == EPI_DSWIGLU || EPI == EPI_DSWIGLU_PACKED) ? 8 : 4);
    kernel<<<num_sms(), threads, SMEM_BYTES, g.stream>>>(
        ta, tb, static_cast<T*>(g.out), g.out_stride, static_cast<T*>(g.aux), g.aux_stride, g.row_map, g.out_peers,
        g.peer_world, g.peer_rows_cap, g.tile_prefix, g.num_experts, static_cast<int>(g.kd), static_cast<int>(g.n),
        idesc, tune_word() | g.tune_extra, g.device_status);
    return static_cast<int>(cudaGetLastError());
}

template <typename T>
static int rows_dispatch(const RowsGemmArgs& g, const CUtensorMap& ta, const CUtensorMap& tb) {
#define XMA_ROWS_CASE(WL, EPI) \
    if (g.w_layout == WL && g.epilogue == EPI) return launch_rows<T, WL, EPI>(g, ta, tb)
    XMA_ROWS_CASE(W_NK, EPI_PLAIN);
    XMA_ROWS_CASE(W_NK, EPI_SWIGLU);
    XMA_ROWS_CASE(W_KN, EPI_PLAIN);
    XMA_ROWS_CASE(W_KN, EPI_DSWIGLU);
    XMA_ROWS_CASE(W_NK, EPI_SWIGLU_PACKED);
    XMA_ROWS_CASE(W_KN, EPI_DSWIGLU_PACKED);
    XMA_ROWS_CASE(W_NK, EPI_PLAIN_PEER);
    XMA_ROWS_CASE(W_KN, EPI_PLAIN_PEER);
#undef XMA_ROWS_CASE
    return XMA_ERR_UNSUPPORTED;
}

}  // namespace tc

bool rows_gemm_tc_supported(const RowsGemmArgs& g) {
    if (g.dtype != XMA_BF16 && g.dtype != XMA_F16) return false;
    if (!tc::device_is_sm100() || !tc::encode_fn()) return false;
    if (g.num_experts > tc::MAX_EXPERTS || g.kd <= 0 || g.n <= 0) return false;
    if (g.kd % 8 || g.n % 8 || g.a_stride % 8 || g.out_stride % 8) return false;
    if (!is_aligned16(g.a) || !is_aligned16(g.w) || !is_aligned16(g.out)) return false;
    const bool plain = (g.epilogue == EPI_PLAIN || g.epilogue == EPI_PLAIN_PEER);
    const bool combo = (g.w_layout == W_NK && (plain || g.epilogue == EPI_SWIGLU ||
                                               g.epilogue == EPI_SWIGLU_PACKED)) ||
                       (g.w_layout == W_KN && (plain || g.epilogue == EPI_DSWIGLU ||
                                               g.epilogue == EPI_DSWIGLU_PACKED));
    if (!combo) return false;
    if (g.epilogue == EPI_PLAIN_PEER &&
        (!g.row_map || !g.out_peers || g.peer_world <= 0 || g.peer_world > PEER_MAX_RANKS || g.peer_rows_cap <= 0))
        return false;
    if (!plain) {
        if (!g.aux || g.aux_stride % 8 || !is_aligned16(g.aux) || g.row_map) return false;
        if ((g.epilogue == EPI_SWIGLU || g.epilogue == EPI_SWIGLU_PACKED) && (g.n % 16)) return false;
    }
    if (static_cast<int64_t>(g.num_experts) * g.n > 0x7fffffffLL || static_cast<int64_t>(g.num_experts) * g.kd > 0x7fffffffLL ||
        g.tile_cap * XMA_ROW_PAD > 0x7fffffffLL)
        return false;
    return true;
}

int rows_gemm_tc(const RowsGemmArgs& g) {
    if (!rows_gemm_tc_supported(g)) return XMA_ERR_UNSUPPORTED;
    if (g.tile_cap == 0) return XMA_OK;
    CUtensorMap ta, tb;
    const uint64_t rows_cap = static_cast<uint64_t>(g.tile_cap) * XMA_ROW_PAD;
    if (!tc::cached_map(&ta, g.dtype, g.a, g.kd, rows_cap, g.a_stride, tc::BM)) return XMA_ERR_TENSOR_MAP;
    bool ok;
    if (g.w_layout == W_NK)
        ok = tc::cached_map(&tb, g.dtype, g.w, g.kd, static_cast<uint64_t>(g.num_experts) * g.n, g.kd, 128);
    else
        ok = tc::cached_map(&tb, g.dtype, g.w, g.n, static_cast<uint64_t>(g.num_experts) * g.kd, g.n, 64);
    if (!ok) return XMA_ERR_TENSOR_MAP;
    if (g.dtype == XMA_BF16) return tc::rows_dispatch<__nv_bfloat16>(g, ta, tb);
    return tc::rows_dispatch<__half>(g, ta, tb);
}

bool dw_gemm_tc_supported(const DwGemmArgs& g) {
    if (g.dtype != XMA_BF16 && g.dtype != XMA_F16) return false;
    if (!tc::device_is_sm100() || !tc::encode_fn()) return false;
    if (g.m <= 0 || g.n <= 0 || g.m % 8 || g.n % 8 || g.x_stride % 8 || g.y_stride % 8) return false;
    if (!is_aligned16(g.x) || !is_aligned16(g.y) || !is_aligned16(g.dw)) return false;
    if (g.m > 0x7fffffffLL || g.n > 0x7fffffffLL || g.rows_cap <= 0 || g.rows_cap > 0x7fffffffLL) return false;
    return true;
}

int dw_gemm_tc(const DwGemmArgs& g) {
    if (!dw_gemm_tc_supported(g)) return XMA_ERR_UNSUPPORTED;
    if (g.num_experts == 0) return XMA_OK;
    CUtensorMap tx, ty;
    if (!tc::cached_map(&tx, g.dtype, g.x, g.m, g.rows_cap, g.x_stride, 64)) return XMA_ERR_TENSOR_MAP;
    if (!tc::cached_map(&ty, g.dtype, g.y, g.n, g.rows_cap, g.y_stride, 64)) return XMA_ERR_TENSOR_MAP;
    const uint32_t idesc = tc::make_idesc(g.dtype, true, true);
    if (g.dtype == XMA_BF16) {
        auto kernel = tc::dw_gemm_tc_kernel<__nv_bfloat16>;
        int rc = tc::set_smem(kernel);
        if (rc) return rc;
        kernel<<<num_sms(), tc::block_threads(4), tc::SMEM_BYTES, g.stream>>>(
            tx, ty, g.counts, g.pad_offsets, g.num_experts, static_cast<int>(g.m), static_cast<int>(g.n),
            static_cast<__nv_bfloat16*>(g.dw), idesc, g.device_status);
    } else {
        auto kernel = tc::dw_gemm_tc_kernel<__half>;
        int rc = tc::set_smem(kernel);
        if (rc) return rc;
        kernel<<<num_sms(), tc::block_threads(4), tc::SMEM_BYTES, g.stream>>>(
            tx, ty, g.counts, g.pad_offsets, g.num_experts, static_cast<int>(g.m), static_cast<int>(g.n),
            static_cast<__half*>(g.dw), idesc, g.device_status);
    }
    return static_cast<int>(cudaGetLastError());
}

}  // namespace xma
