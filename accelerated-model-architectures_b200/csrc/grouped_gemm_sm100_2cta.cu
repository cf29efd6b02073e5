// Two-CTA (cta_group::2) variant of the tcgen05 grouped GEMMs: a pair of CTAs on neighbouring SMs
// computes one 256 x 256 output tile. Each CTA stages its own 128 rows of A and only HALF of the B
// tile (128 of the 256 columns); the tensor cores of both SMs read both halves. Per 64-deep reduction
// block a CTA therefore pulls 32 KiB from L2 instead of 48 KiB (one third less L2->SM traffic and
// shared-memory fill per FLOP than the one-CTA kernel) and the ring holds 6 stages instead of 4.
//
// Protocol (rank 0 = leader of the pair):
//   producers (both CTAs)  : wait own empty[s] -> TMA A/B into own shared memory, completion bytes
//                            are posted to the LEADER's full[s] (cp.async.bulk.tensor .cta_group::2)
//   MMA (leader, one lane) : wait full[s] (expects the bytes of both CTAs) -> tcgen05.mma.cta_group::2
//                            -> tcgen05.commit to empty[s] / acc_full[buf] of BOTH CTAs
//   epilogue (both CTAs)   : wait own acc_full[buf] -> read own 128 accumulator lanes -> one arrive
//                            per warp on the LEADER's acc_empty[buf]
// No TMA load uses cluster multicast. Every wait is bounded as in the one-CTA kernel; both CTAs meet
// at a cluster barrier before tensor memory is released.
#include "sm100_common.cuh"

namespace xma {
namespace tc2 {

using namespace tc;

constexpr int STAGES2 = 6;
constexpr int A2_BYTES = BM * BK * 2;         // 128 rows x 64: 16 KiB
constexpr int B2_BYTES = (BN / 2) * BK * 2;   // this CTA's half of the B tile: 16 KiB
constexpr int STAGE2_BYTES = A2_BYTES + B2_BYTES;
constexpr size_t SMEM2_BYTES = 1024 + static_cast<size_t>(STAGES2) * STAGE2_BYTES +
                               2 * (MAX_EXPERTS + 1) * sizeof(int) + 256 + PEER_STAGE_BYTES;

// Staged SwiGLU-backward epilogue (EPI_DSWIGLU_STAGED): every epilogue warp owns two 4 KiB buffers, each holding
// the gate and the up values of its 32 rows x 32 columns (two TMA boxes, 64-byte swizzle). The room comes from the
// staging of the peer epilogue, which this variant does not use, and from expert tables sized for at most
// STAGED_MAX_EXPERTS experts.
constexpr int STAGED_MAX_EXPERTS = 192;
constexpr int GU_BOX_COLS = 32;
constexpr int GU_HALF_BYTES = 32 * GU_BOX_COLS * 2;  // 32 rows x 32 columns of 16-bit values: 2 KiB
constexpr int GU_BUF_BYTES = 2 * GU_HALF_BYTES;      // gate | up
constexpr int GU_WARP_BYTES = 2 * GU_BUF_BYTES;      // two buffers per epilogue warp
constexpr int GU_STAGE_BYTES = 4 * GU_WARP_BYTES;    // four epilogue warps: 32 KiB
constexpr int GU_PREFETCH_CHUNKS = 3;                // chunks asked for in L2 ahead of the chunk being loaded
constexpr size_t SMEM2_STAGED_BYTES = 1024 + GU_STAGE_BYTES + static_cast<size_t>(STAGES2) * STAGE2_BYTES +
                                      2 * (STAGED_MAX_EXPERTS + 1) * sizeof(int) + 256 + 64;
static_assert(SMEM2_STAGED_BYTES <= 227 * 1024, "staged epilogue: shared memory");

// ---- cluster / pair PTX ---------------------------------------------------------------------------------

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}

__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// shared::cluster address of the same shared-memory location in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local_addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank));
    return r;
}

// TMA load into this CTA's shared memory; the completion bytes go to the mbarrier at `mbar_cluster_addr`,
// which may live in the peer CTA.
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* map, uint32_t mbar_cluster_addr,
                                                 int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4}], [%2];"
        :
        : "r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(mbar_cluster_addr), "r"(c0), "r"(c1)
        : "memory");
}

__device__ __forceinline__ void mbar_arrive_cluster(uint32_t mbar_cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(mbar_cluster_addr) : "memory");
}

__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_result, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
                 "r"(cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}

// D[tmem of both CTAs] (+)= A * B^T, 256 x 256 x 16, issued by one thread of the leader CTA.
__device__ __forceinline__ void umma_f16_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                              uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t"
        "}"
        :
        : "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}

// The mbarrier at this shared-memory offset in BOTH CTAs of the pair gets one arrival once every
// tcgen05.mma issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
    const uint16_t mask = 3;
    asm volatile(
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
            smem_u32(bar)),
        "h"(mask)
        : "memory");
}

template <bool A_MN, bool B_MN>
__device__ __forceinline__ void issue_stage_pair(uint32_t a_saddr, uint32_t b_saddr, uint32_t tmem_d, uint32_t idesc,
                                                 bool first_block) {
    const uint64_t da = smem_desc(a_saddr, A_MN);
    const uint64_t db = smem_desc(b_saddr, B_MN);
#pragma unroll
    for (int k = 0; k < BK / UMMA_K; ++k) {
        umma_f16_pair(tmem_d, da + static_cast<uint64_t>(k * desc_k_step(A_MN)),
                      db + static_cast<uint64_t>(k * desc_k_step(B_MN)), idesc, (first_block && k == 0) ? 0u : 1u);
    }
}

struct Shared2 {
    uint8_t* stage_base;
    int* tile_prefix;  // [E + 1] 128-row tiles in front of each expert
    int* pair_prefix;  // [E + 1] 256-row pair tiles in front of each expert
    uint64_t* full;
    uint64_t* empty;
    uint64_t* acc_full;
    uint64_t* acc_empty;
    uint32_t* tmem_ptr;
    volatile int* abort_flag;
    uint8_t* peer_stage;  // [PEER_STAGE_BYTES], 16-byte aligned (null in the staged SwiGLU-backward variant)
    uint8_t* gu_stage;    // [GU_STAGE_BYTES], 1024-byte aligned (staged SwiGLU-backward variant only)
    uint64_t* gu_full;    // [4 warps][2 buffers] (staged SwiGLU-backward variant only)
};

template <bool STAGED = false>
__device__ __forceinline__ Shared2 carve_smem2(uint8_t* raw) {
    Shared2 s;
    const uint32_t a = smem_u32(raw);
    uint8_t* base = raw + ((1024u - (a & 1023u)) & 1023u);
    constexpr int TABLE = (STAGED ? STAGED_MAX_EXPERTS : MAX_EXPERTS) + 1;
    s.gu_stage = STAGED ? base : nullptr;
    if (STAGED) base += GU_STAGE_BYTES;
    s.stage_base = base;
    uint8_t* p = base + static_cast<size_t>(STAGES2) * STAGE2_BYTES;
    s.tile_prefix = reinterpret_cast<int*>(p);
    p += TABLE * sizeof(int);
    s.pair_prefix = reinterpret_cast<int*>(p);
    p += TABLE * sizeof(int);
    p = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(p) + 7) & ~static_cast<uintptr_t>(7));
    s.full = reinterpret_cast<uint64_t*>(p);
    s.empty = s.full + STAGES2;
    s.acc_full = s.empty + STAGES2;
    s.acc_empty = s.acc_full + 2;
    s.tmem_ptr = reinterpret_cast<uint32_t*>(s.acc_empty + 2);
    s.abort_flag = reinterpret_cast<volatile int*>(s.tmem_ptr + 1);
    uint8_t* tail = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(s.tmem_ptr + 2) + 15) &
                                               ~static_cast<uintptr_t>(15));
    s.peer_stage = STAGED ? nullptr : tail;
    s.gu_full = STAGED ? reinterpret_cast<uint64_t*>(tail) : nullptr;
    return s;
}

// Barriers + tensor-memory allocation of the pair. Must be called by all threads of both CTAs.
__device__ __forceinline__ uint32_t prologue2(const Shared2& s, int warp) {
    if (threadIdx.x == 0) {
        const uint32_t epi_warps = (blockDim.x - 64) >> 5;
        for (int i = 0; i < STAGES2; ++i) {
            mbar_init(&s.full[i], 1);   // the leader's own producer; bytes of both CTAs
            mbar_init(&s.empty[i], 1);  // one commit from the leader's MMA thread
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&s.acc_full[i], 1);
            mbar_init(&s.acc_empty[i], 2 * epi_warps);  // one arrival per epilogue warp of both CTAs
        }
        if (s.gu_full)
            for (int i = 0; i < 8; ++i) mbar_init(&s.gu_full[i], 1);  // lane 0 of the owning warp; bytes of two boxes
        *s.abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tmem_alloc_pair(s.tmem_ptr, TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();  // the peer's barriers exist before anything is posted to them
    tc_fence_after();
    return *s.tmem_ptr;
}

__device__ __forceinline__ void teardown2(const Shared2& s, uint32_t tmem_base, int warp, int* status) {
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();  // neither CTA leaves while the other may still touch its shared or tensor memory
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc_pair(tmem_base, TMEM_COLS);
    }
    if (threadIdx.x == 0 && *s.abort_flag && status) atomicOr(status, XMA_DEV_WAIT_TIMEOUT);
}

// largest e with prefix[e] * n_tiles <= w
__device__ __forceinline__ int find_expert(const int* prefix, int E, int n_tiles, int64_t w) {
    int lo = 0, hi = E;
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (static_cast<int64_t>(prefix[mid]) * n_tiles <= w) lo = mid;
        else hi = mid;
    }
    return lo;
}

struct PairWork {
    int e, n_tile, m_tile;  // m_tile: this CTA's 128-row tile (global index in the padded layout)
    bool active;            // false: this CTA's half lies beyond the expert's rows
};

constexpr int PAIR_RASTER_GROUP = 8;

__device__ __forceinline__ PairWork decode_pair(const Shared2& s, int E, int n_tiles, int64_t w, int rank) {
    PairWork r;
    r.e = find_expert(s.pair_prefix, E, n_tiles, w);
    const int64_t local = w - static_cast<int64_t>(s.pair_prefix[r.e]) * n_tiles;
    const int pt = s.pair_prefix[r.e + 1] - s.pair_prefix[r.e];
    int pm;
    raster_tile(local, pt, n_tiles, PAIR_RASTER_GROUP, pm, r.n_tile);  // 74 pairs: about 8 pair rows x 9 column tiles
    const int mt = s.tile_prefix[r.e + 1] - s.tile_prefix[r.e];
    r.m_tile = s.tile_prefix[r.e] + 2 * pm + rank;
    r.active = (2 * pm + rank) < mt;
    return r;
}

// ======================================================================================================
// Rows GEMM, CTA pair
// ======================================================================================================
template <typename T, int WL, int EPI>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THREADS, 1)
rows_gemm_tc2_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                     const __grid_constant__ CUtensorMap tm_gu, const __grid_constant__ CUtensorMap tm_dgu,
                     T* __restrict__ out, int64_t out_stride, T* __restrict__ aux, int64_t aux_stride,
                     const int* __restrict__ row_map, void* const* __restrict__ out_peers, int peer_world,
                     int64_t peer_rows_cap, const int* __restrict__ g_tile_prefix, int E, int kd, int n,
                     uint32_t idesc, uint32_t tune, int* __restrict__ status) {
    extern __shared__ __align__(16) uint8_t smem_raw[];
    constexpr bool STAGED =
        (EPI == EPI_DSWIGLU_STAGED || EPI == EPI_SWIGLU_STAGED || EPI == EPI_DSWIGLU_PACKED_STAGED);
    constexpr bool IS_SWIGLU = (EPI == EPI_SWIGLU || EPI == EPI_SWIGLU_STAGED);
    const Shared2 s = carve_smem2<STAGED>(smem_raw);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int rank = static_cast<int>(cluster_ctarank());
    const int64_t pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;

    for (int i = threadIdx.x; i <= E; i += blockDim.x) s.tile_prefix[i] = g_tile_prefix[i];
    __syncthreads();
    if (threadIdx.x == 32) {
        int run = 0;
        const int round_up = (tune & TUNE_WHOLE_PAIRS_ONLY) ? 0 : 1;  // an odd last tile: half a pair, or left out
        for (int e = 0; e < E; ++e) {
            s.pair_prefix[e] = run;
            run += (s.tile_prefix[e + 1] - s.tile_prefix[e] + round_up) >> 1;
        }
        s.pair_prefix[E] = run;
    }
    const uint32_t tmem_base = prologue2(s, warp);

    constexpr bool B_MN = (WL == W_KN);
    const int half_n = n / 2;
    const int n_tiles = IS_SWIGLU ? (half_n + 127) / 128 : (n + BN - 1) / BN;
    const int k_blocks = (kd + BK - 1) / BK;
    const int64_t total = static_cast<int64_t>(s.pair_prefix[E]) * n_tiles;

    if (warp == 0) {
        if (lane == 0) {
            // box coordinates of one reduction block; `load` = false only asks for the boxes in L2
            auto boxes = [&](const PairWork& wk, int kb, bool load, uint8_t* sa, uint8_t* sb, uint32_t full0) {
                const bool want_a = load || ((tune & TUNE_PREFETCH_A) && wk.active);
                const bool want_b = load || (tune & TUNE_PREFETCH_B);
                if (want_a) {
                    if (load) tma_load_2d_pair(sa, &tm_a, full0, kb * BK, wk.m_tile * BM);
                    else tma_prefetch_2d(&tm_a, kb * BK, wk.m_tile * BM);
                }
                if (!want_b) return;
                if (!B_MN) {
                    // weight stored [E * n, kd]: this CTA's 128 rows of the 256-row B tile
                    int r0;
                    if (IS_SWIGLU) r0 = wk.e * n + wk.n_tile * 128 + rank * half_n;  // gate | up rows
                    else r0 = wk.e * n + wk.n_tile * BN + rank * 128;
                    if (load) tma_load_2d_pair(sb, &tm_b, full0, kb * BK, r0);
                    else tma_prefetch_2d(&tm_b, kb * BK, r0);
                } else {
                    // weight stored [E * kd, n]: two boxes of 64 columns x 64 reduction rows
#pragma unroll
                    for (int j = 0; j < 2; ++j) {
                        const int c0 = wk.n_tile * BN + rank * 128 + j * 64, c1 = wk.e * kd + kb * BK;
                        if (load) tma_load_2d_pair(sb + j * CHUNK_BYTES, &tm_b, full0, c0, c1);
                        else tma_prefetch_2d(&tm_b, c0, c1);
                    }
                }
            };
            // L2 prefetch cursor: runs `ahead` reduction blocks in front of the loads, across tiles
            const int ahead = static_cast<int>(tune_prefetch_distance(tune));
            int64_t w_pf = pair;
            int kb_pf = 0;
            bool pf_on = ahead > 0 && w_pf < total;
            PairWork wk_pf;
            if (pf_on) wk_pf = decode_pair(s, E, n_tiles, w_pf, rank);
            auto prefetch_step = [&]() {
                if (!pf_on) return;
                boxes(wk_pf, kb_pf, false, nullptr, nullptr, 0u);
                if (++kb_pf == k_blocks) {
                    kb_pf = 0;
                    w_pf += num_pairs;
                    pf_on = w_pf < total;
                    if (pf_on) wk_pf = decode_pair(s, E, n_tiles, w_pf, rank);
                }
            };
            for (int i = 0; i < ahead; ++i) prefetch_step();
            uint32_t it = 0;
            for (int64_t w = pair; w < total; w += num_pairs) {
                const PairWork wk = decode_pair(s, E, n_tiles, w, rank);
                bool ok = true;
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const int st = it % STAGES2;
                    ok = mbar_wait(&s.empty[st], ((it / STAGES2) & 1u) ^ 1u, s.abort_flag);
                    if (!ok) break;
                    uint8_t* sa = s.stage_base + static_cast<size_t>(st) * STAGE2_BYTES;
                    const uint32_t full0 = map_to_cta(smem_u32(&s.full[st]), 0);
                    if (rank == 0) mbar_expect_tx(&s.full[st], 2 * STAGE2_BYTES);
                    boxes(wk, kb, true, sa, sa + A2_BYTES, full0);
                    prefetch_step();
                }
                if (!ok) break;
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            uint32_t it = 0, lt = 0;
            for (int64_t w = pair; w < total; w += num_pairs, ++lt) {
                const uint32_t buf = lt & 1u;
                if (!mbar_wait(&s.acc_empty[buf], ((lt >> 1) & 1u) ^ 1u, s.abort_flag)) break;
                tc_fence_after();
                const uint32_t tmem_d = tmem_base + buf * BN;
                bool ok = true;
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const int st = it % STAGES2;
                    ok = mbar_wait(&s.full[st], (it / STAGES2) & 1u, s.abort_flag);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t sa = smem_u32(s.stage_base + static_cast<size_t>(st) * STAGE2_BYTES);
                    issue_stage_pair<false, B_MN>(sa, sa + A2_BYTES, tmem_d, idesc, kb == 0);
                    umma_commit_pair(&s.empty[st]);
                }
                if (!ok) break;
                umma_commit_pair(&s.acc_full[buf]);
            }
        }
    } else if constexpr (EPI == EPI_SWIGLU_STAGED) {
        // SwiGLU forward with its three outputs (gate and up, rounded to the storage type, and the activation) leaving
        // by TMA stores: a thread owns an accumulator row, so direct stores are 32 rows x 16 bytes per instruction,
        // twelve of them per 32 gate columns. The warp writes its 32 x 32 boxes into shared memory instead (64-byte
        // swizzle, 6 KiB per warp) and lane 0 hands them to the TMA unit; the buffer is reused once that store has
        // read it, which it has normally done while the next chunk was computed.
        // Four epilogue warps; the activation width is a multiple of 32.
        const int quarter = warp & 3;
        uint8_t* wst = s.gu_stage + (warp - 2) * GU_WARP_BYTES;
        uint32_t lt = 0;
        for (int64_t w = pair; w < total; w += num_pairs, ++lt) {
            const PairWork wk = decode_pair(s, E, n_tiles, w, rank);
            const uint32_t buf = lt & 1u;
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + buf * BN;
            const int row0 = wk.m_tile * BM + quarter * 32;
            const int j0 = wk.n_tile * 128;
            const int nch = min(4, (half_n - j0) / GU_BOX_COLS);
            if (!mbar_wait_epilogue(&s.acc_full[buf], (lt >> 1) & 1u, s.abort_flag)) break;
            tc_fence_after();
            if (wk.active) {
#pragma unroll 1
                for (int c = 0; c < nch; ++c) {
                    uint32_t g[32], u[32];
                    tmem_ld32(taddr + c * 32, g);
                    tmem_ld32(taddr + 128 + c * 32, u);
                    tmem_ld_wait();
                    uint4 qg[4], qu[4], qa[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        float gr[8], ur[8], ac[8];
#pragma unroll
                        for (int t = 0; t < 8; ++t) {
                            gr[t] = round_to<T>(__uint_as_float(g[8 * i + t]));
                            ur[t] = round_to<T>(__uint_as_float(u[8 * i + t]));
                            ac[t] = ur[t] * gr[t] * fast_sigmoid(gr[t]);
                        }
                        qg[i] = pack8<T>(gr);
                        qu[i] = pack8<T>(ur);
                        qa[i] = pack8<T>(ac);
                    }
                    if (lane == 0) tma_store_wait_read();  // the previous chunk's store has read the buffer
                    __syncwarp();
                    uint8_t* bp = wst + lane * (GU_BOX_COLS * 2);
                    const int sw = (lane >> 1) & 3;
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        *reinterpret_cast<uint4*>(bp + ((i ^ sw) << 4)) = qg[i];
                        *reinterpret_cast<uint4*>(bp + GU_HALF_BYTES + ((i ^ sw) << 4)) = qu[i];
                        *reinterpret_cast<uint4*>(bp + 2 * GU_HALF_BYTES + ((i ^ sw) << 4)) = qa[i];
                    }
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) {
                        const int col = j0 + c * GU_BOX_COLS;
                        tma_store_2d(&tm_gu, wst, col, row0);
                        tma_store_2d(&tm_gu, wst + GU_HALF_BYTES, half_n + col, row0);
                        tma_store_2d(&tm_dgu, wst + 2 * GU_HALF_BYTES, col, row0);
                        tma_store_commit();
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&s.acc_empty[buf]), 0));
        }
        if (lane == 0) tma_store_wait_all();
    } else if constexpr (STAGED) {
        // SwiGLU backward with gate|up and d gate|d up moved by TMA, 32 columns at a time. A thread owns one
        // accumulator row, so reading gate|up of that row straight from global memory costs a warp 32 rows x 16
        // bytes per instruction (32 L1 wavefronts, and a DRAM latency per 32-column chunk whenever the L2 prefetch
        // of a whole tile ahead had been evicted again: 0.76 PFLOP/s where the other GEMMs of the 64-expert layer
        // reach 1.15-1.37). Here lane 0 of each warp asks the TMA unit for the warp's 32 x 32 gate and up boxes of
        // the next two chunks (and, in L2, of the chunks behind them) while the warp works on the current one out
        // of shared memory (64-byte swizzle: a row's four 16-byte pieces sit at piece ^ ((row >> 1) & 3), conflict-free
        // for one row per lane); the results overwrite the chunk in place and leave by a TMA store.
        // Four epilogue warps; the activation width is a multiple of 32.
        const int quarter = warp & 3;
        uint8_t* wst = s.gu_stage + (warp - 2) * GU_WARP_BYTES;
        uint64_t* wbar = s.gu_full + (warp - 2) * 2;
        // Interleaved layout (gate, up, gate, up, ... along the columns): the 32 activation columns of a chunk are
        // one box of 64 columns (128-byte swizzle: a row's eight 16-byte pieces sit at piece ^ (row & 7)).
        constexpr bool PACKED = (EPI == EPI_DSWIGLU_PACKED_STAGED);
        auto chunk_boxes = [&](bool load, uint32_t qi, int64_t row, int col) {  // lane 0
            if (load) {
                uint8_t* dst = wst + (qi & 1u) * GU_BUF_BYTES;
                mbar_expect_tx(&wbar[qi & 1u], GU_BUF_BYTES);
                if (PACKED) {
                    tma_load_2d(dst, &tm_gu, &wbar[qi & 1u], 2 * col, static_cast<int>(row));
                } else {
                    tma_load_2d(dst, &tm_gu, &wbar[qi & 1u], col, static_cast<int>(row));
                    tma_load_2d(dst + GU_HALF_BYTES, &tm_gu, &wbar[qi & 1u], n + col, static_cast<int>(row));
                }
            } else if (PACKED) {
                tma_prefetch_2d(&tm_gu, 2 * col, static_cast<int>(row));
            } else {
                tma_prefetch_2d(&tm_gu, col, static_cast<int>(row));
                tma_prefetch_2d(&tm_gu, n + col, static_cast<int>(row));
            }
        };
        auto chunks_of = [&](const PairWork& t) { return min(BN / GU_BOX_COLS, (n - t.n_tile * BN) / GU_BOX_COLS); };
        uint32_t q = 0;  // chunks this warp has taken: buffer q & 1, barrier phase (q >> 1) & 1
        int ahead = 0;   // lane 0: chunks q, q + 1, ... already requested (at most 2: one per buffer)
        uint32_t lt = 0;
        for (int64_t w = pair; w < total; w += num_pairs, ++lt) {
            const PairWork wk = decode_pair(s, E, n_tiles, w, rank);
            const uint32_t buf = lt & 1u;
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + buf * BN;
            const int64_t row0 = static_cast<int64_t>(wk.m_tile) * BM + quarter * 32;
            const int n0 = wk.n_tile * BN;
            const int nch = chunks_of(wk);
            bool ok = true;
            if (wk.active) {
                PairWork nx = wk;
                bool has_next = w + num_pairs < total;
                if (has_next) {
                    nx = decode_pair(s, E, n_tiles, w + num_pairs, rank);
                    has_next = nx.active;
                }
                const int64_t nx_row0 = static_cast<int64_t>(nx.m_tile) * BM + quarter * 32;
                const int nx_nch = has_next ? chunks_of(nx) : 0;
                // chunk `cc` of the stream that starts at this tile's chunk 0 and runs on into the next tile
                auto stream_chunk = [&](bool load, uint32_t qi, int cc) -> bool {
                    if (cc < nch) chunk_boxes(load, qi, row0, n0 + cc * GU_BOX_COLS);
                    else if (cc - nch < nx_nch) chunk_boxes(load, qi, nx_row0, nx.n_tile * BN + (cc - nch) * GU_BOX_COLS);
                    else return false;
                    return true;
                };
                if (lane == 0) {
                    if (ahead == 0) tma_store_wait_read();  // (both buffers may still feed stores of an earlier tile)
                    while (ahead < 2 && stream_chunk(true, q + ahead, ahead)) ++ahead;
                    for (int cc = 2; cc < 2 + GU_PREFETCH_CHUNKS; ++cc) stream_chunk(false, 0u, cc);
                }
                ok = mbar_wait_epilogue(&s.acc_full[buf], (lt >> 1) & 1u, s.abort_flag);
                tc_fence_after();
#pragma unroll 1
                for (int c = 0; ok && c < nch; ++c, ++q) {
                    ok = mbar_wait(&wbar[q & 1u], (q >> 1) & 1u, s.abort_flag);
                    if (!ok) break;
                    uint32_t v[32];
                    tmem_ld32(taddr + c * 32, v);
                    if constexpr (PACKED) {
                        uint8_t* bp = wst + (q & 1u) * GU_BUF_BYTES + lane * (GU_BOX_COLS * 4);
                        const int sw = lane & 7;
                        uint4 pq[8];
#pragma unroll
                        for (int i = 0; i < 8; ++i) pq[i] = *reinterpret_cast<const uint4*>(bp + ((i ^ sw) << 4));
                        tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < 8; ++i) {  // 4 activation columns = 8 interleaved values
                            float gu[8], dd[8];
                            unpack8<T>(pq[i], gu);
#pragma unroll
                            for (int t = 0; t < 4; ++t) {
                                const float d = __uint_as_float(v[4 * i + t]);
                                const float g = gu[2 * t], u = gu[2 * t + 1];
                                const float sg = fast_sigmoid(g);
                                dd[2 * t] = d * u * sg * (1.0f + g * (1.0f - sg));
                                dd[2 * t + 1] = d * g * sg;
                            }
                            *reinterpret_cast<uint4*>(bp + ((i ^ sw) << 4)) = pack8<T>(dd);
                        }
                    } else {
                        uint8_t* bp = wst + (q & 1u) * GU_BUF_BYTES + lane * (GU_BOX_COLS * 2);
                        const int sw = (lane >> 1) & 3;
                        uint4 gq[4], uq[4];
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            gq[i] = *reinterpret_cast<const uint4*>(bp + ((i ^ sw) << 4));
                            uq[i] = *reinterpret_cast<const uint4*>(bp + GU_HALF_BYTES + ((i ^ sw) << 4));
                        }
                        tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            float gg[8], uu[8], dg[8], du[8];
                            unpack8<T>(gq[i], gg);
                            unpack8<T>(uq[i], uu);
#pragma unroll
                            for (int t = 0; t < 8; ++t) {
                                const float d = __uint_as_float(v[8 * i + t]);
                                const float sg = fast_sigmoid(gg[t]);
                                dg[t] = d * uu[t] * sg * (1.0f + gg[t] * (1.0f - sg));
                                du[t] = d * gg[t] * sg;
                            }
                            *reinterpret_cast<uint4*>(bp + ((i ^ sw) << 4)) = pack8<T>(dg);
                            *reinterpret_cast<uint4*>(bp + GU_HALF_BYTES + ((i ^ sw) << 4)) = pack8<T>(du);
                        }
                    }
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) {
                        const uint8_t* src = wst + (q & 1u) * GU_BUF_BYTES;
                        if (PACKED) {
                            tma_store_2d(&tm_dgu, src, 2 * (n0 + c * GU_BOX_COLS), static_cast<int>(row0));
                        } else {
                            tma_store_2d(&tm_dgu, src, n0 + c * GU_BOX_COLS, static_cast<int>(row0));
                            tma_store_2d(&tm_dgu, src + GU_HALF_BYTES, n + n0 + c * GU_BOX_COLS,
                                         static_cast<int>(row0));
                        }
                        tma_store_commit();
                        // this buffer takes the chunk after next as soon as the store has read it
                        --ahead;
                        tma_store_wait_read();
                        while (ahead < 2 && stream_chunk(true, q + 1 + ahead, c + 1 + ahead)) ++ahead;
                        stream_chunk(false, 0u, c + 3 + GU_PREFETCH_CHUNKS - 1);
                    }
                }
            } else {
                ok = mbar_wait_epilogue(&s.acc_full[buf], (lt >> 1) & 1u, s.abort_flag);
            }
            if (!ok) break;
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&s.acc_empty[buf]), 0));
        }
        if (lane == 0) tma_store_wait_all();
    } else {
        const int quarter = warp & 3;
        const int parts = (static_cast<int>(blockDim.x) - 64) >> 7;
        const int part = (warp - 2) >> 2;
        const int chunks = (BN / 32) / parts;
        const int row_in_tile = quarter * 32 + lane;
        // one staging region per epilogue warp when there are four of them
        uint8_t* peer_stage = (parts == 1) ? s.peer_stage + (warp - 2) * PEER_STAGE_WARP_BYTES : nullptr;
        uint32_t lt = 0;
        for (int64_t w = pair; w < total; w += num_pairs, ++lt) {
            const PairWork wk = decode_pair(s, E, n_tiles, w, rank);
            const uint32_t buf = lt & 1u;
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + buf * BN;
            const int64_t r = static_cast<int64_t>(wk.m_tile) * BM + row_in_tile;
            if ((EPI == EPI_DSWIGLU || EPI == EPI_DSWIGLU_PACKED) && (tune & TUNE_GU_PREFETCH) &&
                w + num_pairs < total) {
                const PairWork nx = decode_pair(s, E, n_tiles, w + num_pairs, rank);
                if (nx.active)
                    prefetch_gate_up<T, EPI>(aux, aux_stride, static_cast<int64_t>(nx.m_tile) * BM + row_in_tile,
                                             nx.n_tile, n, part, chunks);
            }
            if (!rows_epilogue_tile<T, EPI>(&s.acc_full[buf], (lt >> 1) & 1u, s.abort_flag, taddr, r, wk.active,
                                            wk.n_tile, n, half_n, out, out_stride, aux, aux_stride, row_map, out_peers,
                                            peer_world, peer_rows_cap, status, peer_stage, part, chunks))
                break;
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&s.acc_empty[buf]), 0));
        }
    }
    teardown2(s, tmem_base, warp, status);
}

// ======================================================================================================
// Weight-gradient GEMM, CTA pair: 256 x 256 tile of dW_e; CTA `rank` owns rows [128 * rank, +128) of it
// and stages columns [128 * rank, +128) of the Y operand.
//
// Work hand-out. A tile of dW_e costs as much as expert e has rows, and loads are anything but equal (a Zipf-
// skewed router gives some experts ten times the mean and some nothing), so with DYN the pairs do not walk a
// fixed stride through the tiles: experts are ranked by row count, tiles are numbered heaviest expert first,
// and a pair takes the next number from an atomic ticket whenever it starts a tile (longest-processing-time
// order: the light tiles at the end level the finish line). The leader's producer thread draws the ticket;
// the other roles of the pair (the second CTA's producer, the MMA thread, the epilogue warps of both CTAs)
// run at their own pace behind it, so the drawn numbers are handed on through a small ring per pair in
// global memory: one 64-bit word per entry, (sequence number + 1) << 32 | tile number, written with release
// and polled with acquire semantics - tag and payload in one word, no separate flag. A consumer is at most
// 8 tiles behind the producer (6 ring stages of at least one reduction block each, 2 accumulator buffers), the
// ring holds 16. Experts without rows get their zeros from the epilogue warps up front and take no ticket.
// Every poll is bounded like the mbarrier waits.
// ======================================================================================================
constexpr int SCHED_RING = 16;
constexpr int SCHED_MAX_PAIRS = 128;
constexpr int SCHED_SLOTS = 16;  // launches that may be in flight on one device, each with its own ticket and rings
constexpr uint32_t SCHED_END = 0xffffffffu;

struct DwSched {
    unsigned long long ring[SCHED_MAX_PAIRS][SCHED_RING];
    unsigned ticket;
    unsigned pad[31];
};

static __device__ DwSched g_dw_sched[SCHED_SLOTS];

__device__ __forceinline__ void sched_publish(DwSched* sc, int64_t pair, uint32_t seq, uint32_t value) {
    const unsigned long long word = (static_cast<unsigned long long>(seq + 1u) << 32) | value;
    asm volatile("st.release.gpu.global.u64 [%0], %1;" ::"l"(&sc->ring[pair][seq % SCHED_RING]), "l"(word) : "memory");
}

// False when the bounded wait gave up (the CTA-wide abort flag is raised then).
__device__ __forceinline__ bool sched_fetch(const DwSched* sc, int64_t pair, uint32_t seq, volatile int* abort_flag,
                                            uint32_t& value) {
    const unsigned long long* p = &sc->ring[pair][seq % SCHED_RING];
    const unsigned long long t0 = globaltimer_ns();
    uint32_t spins = 0;
    for (;;) {
        unsigned long long v;
        asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
        if (static_cast<uint32_t>(v >> 32) == seq + 1u) {
            value = static_cast<uint32_t>(v);
            return true;
        }
        if ((++spins & 0x3fu) == 0u) {
            if (*abort_flag) return false;
            if (globaltimer_ns() - t0 > WAIT_LIMIT_NS) {
                *abort_flag = 1;
                return false;
            }
        }
    }
}

template <typename T, bool DYN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THREADS, 1)
dw_gemm_tc2_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_y,
                   const uint32_t* __restrict__ counts, const int* __restrict__ pad_offsets, int E, int m, int n,
                   T* __restrict__ dw, uint32_t idesc, uint32_t tune, DwSched* __restrict__ sched,
                   int* __restrict__ status) {
    extern __shared__ __align__(16) uint8_t smem_raw[];
    const Shared2 s = carve_smem2(smem_raw);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int rank = static_cast<int>(cluster_ctarank());
    const int64_t pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;

    const int m_tiles = (m + 2 * BM - 1) / (2 * BM);
    const int n_tiles = (n + BN - 1) / BN;
    const int per_e = m_tiles * n_tiles;

    // DYN: the experts ranked by row count (ties by index), the ones without rows last. s_order[k] = k-th
    // heaviest expert, s_cnt = the counts (the two prefix tables of the rows kernel are free here).
    int* s_cnt = s.pair_prefix;
    int* s_order = s.tile_prefix;
    int n_busy = E;  // experts that have rows
    if (DYN) {
        for (int e = threadIdx.x; e < E; e += blockDim.x) s_cnt[e] = static_cast<int>(counts[e]);
        __syncthreads();
        n_busy = 0;
        for (int base = 0; base < E; base += blockDim.x) {
            const int e = base + threadIdx.x;
            bool busy = false;
            if (e < E) {
                const int c = s_cnt[e];
                busy = c > 0;
                int pos = 0;
                for (int j = 0; j < E; ++j) {
                    const int cj = s_cnt[j];
                    pos += (cj > c || (cj == c && j < e)) ? 1 : 0;
                }
                s_order[pos] = e;
            }
            n_busy += __syncthreads_count(busy);
        }
    }
    const uint32_t tmem_base = prologue2(s, warp);
    const int64_t total = static_cast<int64_t>(n_busy) * per_e;  // DYN: tickets; else every (expert, tile)
    const int64_t total_static = static_cast<int64_t>(E) * per_e;

    // work item of a ticket (DYN) or of a static index
    auto item = [&](int64_t w) {
        DwWork wk = decode_dw(w, m_tiles, n_tiles);
        if (DYN) wk.e = s_order[wk.e];
        return wk;
    };
    auto rows_of = [&](int e) { return DYN ? s_cnt[e] : static_cast<int>(counts[e]); };

    if (warp == 0) {
        if (lane == 0) {
            auto boxes = [&](const DwWork& wk, int row, bool load, uint8_t* sa, uint8_t* sb, uint32_t full0) {
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    const int c0 = wk.m_tile * 2 * BM + rank * BM + j * 64;
                    if (load) tma_load_2d_pair(sa + j * CHUNK_BYTES, &tm_x, full0, c0, row);
                    else if (tune & TUNE_PREFETCH_A) tma_prefetch_2d(&tm_x, c0, row);
                }
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    const int c0 = wk.n_tile * BN + rank * 128 + j * 64;
                    if (load) tma_load_2d_pair(sb + j * CHUNK_BYTES, &tm_y, full0, c0, row);
                    else if (tune & TUNE_PREFETCH_B) tma_prefetch_2d(&tm_y, c0, row);
                }
            };
            uint32_t it = 0;
            auto load_item = [&](const DwWork& wk) {
                const int k_blocks = (rows_of(wk.e) + BK - 1) / BK;
                const int row0 = pad_offsets[wk.e];
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const int st = it % STAGES2;
                    if (!mbar_wait(&s.empty[st], ((it / STAGES2) & 1u) ^ 1u, s.abort_flag)) return false;
                    uint8_t* sa = s.stage_base + static_cast<size_t>(st) * STAGE2_BYTES;
                    const uint32_t full0 = map_to_cta(smem_u32(&s.full[st]), 0);
                    if (rank == 0) mbar_expect_tx(&s.full[st], 2 * STAGE2_BYTES);
                    boxes(wk, row0 + kb * BK, true, sa, sa + A2_BYTES, full0);
                }
                return true;
            };
            if (DYN) {
                for (uint32_t seq = 0;; ++seq) {
                    uint32_t t;
                    if (rank == 0) {  // the pair's scheduler
                        t = atomicAdd(&sched->ticket, 1u);
                        if (t >= total) t = SCHED_END;
                        sched_publish(sched, pair, seq, t);
                    } else if (!sched_fetch(sched, pair, seq, s.abort_flag, t)) {
                        break;
                    }
                    if (t == SCHED_END || !load_item(item(t))) break;
                }
            } else {
                // L2 prefetch cursor, `ahead` reduction blocks in front of the loads (experts without rows have none)
                const int ahead = static_cast<int>(tune_prefetch_distance(tune));
                int64_t w_pf = pair;
                int kb_pf = 0, kbs_pf = 0, row_pf = 0;
                DwWork wk_pf;
                bool pf_on = ahead > 0;
                auto pf_seek = [&]() {  // first work item at or after w_pf that has reduction blocks
                    for (; w_pf < total_static; w_pf += num_pairs) {
                        wk_pf = decode_dw(w_pf, m_tiles, n_tiles);
                        kbs_pf = (static_cast<int>(counts[wk_pf.e]) + BK - 1) / BK;
                        if (kbs_pf > 0) break;
                    }
                    pf_on = w_pf < total_static;
                    if (pf_on) row_pf = pad_offsets[wk_pf.e];
                    kb_pf = 0;
                };
                if (pf_on) pf_seek();
                auto prefetch_step = [&]() {
                    if (!pf_on) return;
                    boxes(wk_pf, row_pf + kb_pf * BK, false, nullptr, nullptr, 0u);
                    if (++kb_pf == kbs_pf) {
                        w_pf += num_pairs;
                        pf_seek();
                    }
                };
                for (int i = 0; i < ahead; ++i) prefetch_step();
                for (int64_t w = pair; w < total_static; w += num_pairs) {
                    const DwWork wk = decode_dw(w, m_tiles, n_tiles);
                    const int k_blocks = (static_cast<int>(counts[wk.e]) + BK - 1) / BK;
                    const int row0 = pad_offsets[wk.e];
                    bool ok = true;
                    for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                        const int st = it % STAGES2;
                        ok = mbar_wait(&s.empty[st], ((it / STAGES2) & 1u) ^ 1u, s.abort_flag);
                        if (!ok) break;
                        uint8_t* sa = s.stage_base + static_cast<size_t>(st) * STAGE2_BYTES;
                        const uint32_t full0 = map_to_cta(smem_u32(&s.full[st]), 0);
                        if (rank == 0) mbar_expect_tx(&s.full[st], 2 * STAGE2_BYTES);
                        boxes(wk, row0 + kb * BK, true, sa, sa + A2_BYTES, full0);
                        prefetch_step();
                    }
                    if (!ok) break;
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            uint32_t it = 0, lt = 0;
            // main loop of one tile with k_blocks >= 1 reduction blocks; false when a bounded wait gave up
            auto mma_item = [&](int k_blocks) {
                const uint32_t buf = lt & 1u;
                if (!mbar_wait(&s.acc_empty[buf], ((lt >> 1) & 1u) ^ 1u, s.abort_flag)) return false;
                tc_fence_after();
                const uint32_t tmem_d = tmem_base + buf * BN;
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const int st = it % STAGES2;
                    if (!mbar_wait(&s.full[st], (it / STAGES2) & 1u, s.abort_flag)) return false;
                    tc_fence_after();
                    const uint32_t sa = smem_u32(s.stage_base + static_cast<size_t>(st) * STAGE2_BYTES);
                    issue_stage_pair<true, true>(sa, sa + A2_BYTES, tmem_d, idesc, kb == 0);
                    umma_commit_pair(&s.empty[st]);
                }
                umma_commit_pair(&s.acc_full[buf]);
                ++lt;
                return true;
            };
            if (DYN) {
                for (uint32_t seq = 0;; ++seq) {
                    uint32_t t;
                    if (!sched_fetch(sched, pair, seq, s.abort_flag, t) || t == SCHED_END) break;
                    if (!mma_item((rows_of(item(t).e) + BK - 1) / BK)) break;
                }
            } else {
                for (int64_t w = pair; w < total_static; w += num_pairs) {
                    const DwWork wk = decode_dw(w, m_tiles, n_tiles);
                    const int k_blocks = (static_cast<int>(counts[wk.e]) + BK - 1) / BK;
                    if (k_blocks == 0) continue;
                    if (!mma_item(k_blocks)) break;
                }
            }
        }
    } else {
        const int quarter = warp & 3;
        const int parts = (static_cast<int>(blockDim.x) - 64) >> 7;
        const int part = (warp - 2) >> 2;
        const int chunks = (BN / 32) / parts;
        const int row_in_tile = quarter * 32 + lane;
        uint32_t lt = 0;
        auto zero_tile = [&](const DwWork& wk) {
            const int row = wk.m_tile * 2 * BM + rank * BM + row_in_tile;
            const int n0 = wk.n_tile * BN;
            if (row >= m) return;
            T* dst = dw + (static_cast<int64_t>(wk.e) * m + row) * n + n0;
            const uint4 z = make_uint4(0u, 0u, 0u, 0u);
            for (int c = part * chunks * 32; c < (part + 1) * chunks * 32 && n0 + c < n; c += 8)
                *reinterpret_cast<uint4*>(dst + c) = z;
        };
        auto store_tile = [&](const DwWork& wk) {
            const int row = wk.m_tile * 2 * BM + rank * BM + row_in_tile;
            const int n0 = wk.n_tile * BN;
            T* dst = dw + (static_cast<int64_t>(wk.e) * m + row) * n + n0;
            const uint32_t buf = lt & 1u;
            if (!mbar_wait_epilogue(&s.acc_full[buf], (lt >> 1) & 1u, s.abort_flag)) return false;
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
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&s.acc_empty[buf]), 0));
            ++lt;
            return true;
        };
        if (DYN) {
            // experts without rows: exact zeros, handed out by a fixed stride (they sit behind the busy ones)
            const int64_t idle_items = static_cast<int64_t>(E - n_busy) * per_e;
            for (int64_t z = pair; z < idle_items; z += num_pairs) zero_tile(item(total + z));
            for (uint32_t seq = 0;; ++seq) {
                uint32_t t = SCHED_END;
                int ok = 1;
                if (lane == 0) ok = sched_fetch(sched, pair, seq, s.abort_flag, t) ? 1 : 0;
                ok = __shfl_sync(0xffffffffu, ok, 0);
                t = __shfl_sync(0xffffffffu, t, 0);
                if (!ok || t == SCHED_END) break;
                if (!store_tile(item(t))) break;
            }
        } else {
            for (int64_t w = pair; w < total_static; w += num_pairs) {
                const DwWork wk = decode_dw(w, m_tiles, n_tiles);
                if (counts[wk.e] == 0u) {
                    zero_tile(wk);
                    continue;
                }
                if (!store_tile(wk)) break;
            }
        }
    }
    teardown2(s, tmem_base, warp, status);
}

// ---- host side ---------------------------------------------------------------------------------------

static int pair_grid() { return num_sms() & ~1; }

template <typename K>
static int set_smem2(K kernel, size_t bytes = SMEM2_BYTES) {
    apply_epilogue_tuning();
    return set_dynamic_smem_once(kernel, bytes);
}

// `tgu` / `tdgu`: maps over aux / out with 32 x 32 boxes for the staged SwiGLU-backward epilogue (any valid map
// for the other variants, which do not touch them).
template <typename T, int WL, int EPI>
static int launch_rows2(const RowsGemmArgs& g, const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tgu,
                        const CUtensorMap& tdgu) {
    constexpr bool STAGED =
        (EPI == EPI_DSWIGLU_STAGED || EPI == EPI_SWIGLU_STAGED || EPI == EPI_DSWIGLU_PACKED_STAGED);
    constexpr size_t SMEM = STAGED ? SMEM2_STAGED_BYTES : SMEM2_BYTES;
    auto kernel = rows_gemm_tc2_kernel<T, WL, EPI>;
    int rc = set_smem2(kernel, SMEM);
    if (rc) return rc;
    const uint32_t idesc = make_idesc_mn(g.dtype, false, WL == W_KN, 2 * BM, BN);
    // (rows bound for other ranks, and the staged SwiGLU backward, are staged per epilogue warp: always four
    // warps then)
    const int threads = (EPI == EPI_PLAIN_PEER || STAGED)
                            ? 64 + 32 * 4
                            : block_threads(4);  // (the SwiGLU-backward epilogue measured 3.6 % faster with 4 warps
                                                 // than with 8 on the dense-expert layer, the others equal)
    kernel<<<pair_grid(), threads, SMEM, g.stream>>>(
        ta, tb, tgu, tdgu, static_cast<T*>(g.out), g.out_stride, static_cast<T*>(g.aux), g.aux_stride, g.row_map,
        g.out_peers, g.peer_world, g.peer_rows_cap, g.tile_prefix, g.num_experts, static_cast<int>(g.kd),
        static_cast<int>(g.n), idesc, tune_word() | g.tune_extra, g.device_status);
    return static_cast<int>(cudaGetLastError());
}

// Whether the SwiGLU backward of these arguments can take the staged epilogue (and builds its two maps: gate|up
// to read, d gate|d up to write).
static bool staged_dswiglu_maps(const RowsGemmArgs& g, CUtensorMap* tgu, CUtensorMap* tdgu) {
    if (g.epilogue != EPI_DSWIGLU || g.w_layout != W_KN || !(tuning().dswiglu_staged & 1)) return false;
    if (g.n % GU_BOX_COLS || g.num_experts > STAGED_MAX_EXPERTS) return false;
    if (g.aux_stride % 8 || g.out_stride % 8 || !is_aligned16(g.aux) || !is_aligned16(g.out)) return false;
    const uint64_t rows_cap = static_cast<uint64_t>(g.tile_cap) * XMA_ROW_PAD;
    return cached_map(tgu, g.dtype, g.aux, 2 * g.n, rows_cap, g.aux_stride, 32, GU_BOX_COLS) &&
           cached_map(tdgu, g.dtype, g.out, 2 * g.n, rows_cap, g.out_stride, 32, GU_BOX_COLS);
}

// The same for the interleaved layout: one box of 64 interleaved columns (128-byte swizzle) per 32 activation columns.
static bool staged_dswiglu_packed_maps(const RowsGemmArgs& g, CUtensorMap* tgu, CUtensorMap* tdgu) {
    if (g.epilogue != EPI_DSWIGLU_PACKED || g.w_layout != W_KN || !(tuning().dswiglu_staged & 1)) return false;
    if (g.n % GU_BOX_COLS || g.num_experts > STAGED_MAX_EXPERTS) return false;
    if (g.aux_stride % 8 || g.out_stride % 8 || !is_aligned16(g.aux) || !is_aligned16(g.out)) return false;
    const uint64_t rows_cap = static_cast<uint64_t>(g.tile_cap) * XMA_ROW_PAD;
    return cached_map(tgu, g.dtype, g.aux, 2 * g.n, rows_cap, g.aux_stride, 32, 64) &&
           cached_map(tdgu, g.dtype, g.out, 2 * g.n, rows_cap, g.out_stride, 32, 64);
}

// The same for the SwiGLU forward (maps: gate|up [rows, n] and the activation [rows, n / 2], both written).
static bool staged_swiglu_maps(const RowsGemmArgs& g, CUtensorMap* tgu, CUtensorMap* tact) {
    if (g.epilogue != EPI_SWIGLU || g.w_layout != W_NK || !(tuning().dswiglu_staged & 2)) return false;
    // Measured against the GEMM of equal work beside it: with a 2048-deep reduction the staged stores make the up
    // projection 7 % faster (the epilogue is then as long as the main loop of a tile); with 4096 they cost 0-5 %
    // (the epilogue hides behind the main loop anyway and its TMA stores queue with the operand loads). Bit 2 of
    // the switch forces the staged stores for any depth.
    if (g.kd >= 4096 && !(tuning().dswiglu_staged & 4)) return false;
    if ((g.n / 2) % GU_BOX_COLS || g.num_experts > STAGED_MAX_EXPERTS) return false;
    if (g.aux_stride % 8 || g.out_stride % 8 || !is_aligned16(g.aux) || !is_aligned16(g.out)) return false;
    const uint64_t rows_cap = static_cast<uint64_t>(g.tile_cap) * XMA_ROW_PAD;
    return cached_map(tgu, g.dtype, g.aux, g.n, rows_cap, g.aux_stride, 32, GU_BOX_COLS) &&
           cached_map(tact, g.dtype, g.out, g.n / 2, rows_cap, g.out_stride, 32, GU_BOX_COLS);
}

template <typename T>
static int rows_dispatch2(const RowsGemmArgs& g, const CUtensorMap& ta, const CUtensorMap& tb) {
    {
        CUtensorMap tgu, tdgu;
        if (staged_dswiglu_maps(g, &tgu, &tdgu)) return launch_rows2<T, W_KN, EPI_DSWIGLU_STAGED>(g, ta, tb, tgu, tdgu);
        if (staged_swiglu_maps(g, &tgu, &tdgu)) return launch_rows2<T, W_NK, EPI_SWIGLU_STAGED>(g, ta, tb, tgu, tdgu);
        if (staged_dswiglu_packed_maps(g, &tgu, &tdgu))
            return launch_rows2<T, W_KN, EPI_DSWIGLU_PACKED_STAGED>(g, ta, tb, tgu, tdgu);
    }
#define XMA_ROWS2_CASE(WL, EPI) \
    if (g.w_layout == WL && g.epilogue == EPI) return launch_rows2<T, WL, EPI>(g, ta, tb, ta, ta)
    XMA_ROWS2_CASE(W_NK, EPI_PLAIN);
    XMA_ROWS2_CASE(W_NK, EPI_SWIGLU);
    XMA_ROWS2_CASE(W_KN, EPI_PLAIN);
    XMA_ROWS2_CASE(W_KN, EPI_DSWIGLU);
    XMA_ROWS2_CASE(W_NK, EPI_SWIGLU_PACKED);
    XMA_ROWS2_CASE(W_KN, EPI_DSWIGLU_PACKED);
    XMA_ROWS2_CASE(W_NK, EPI_PLAIN_PEER);
    XMA_ROWS2_CASE(W_KN, EPI_PLAIN_PEER);
#undef XMA_ROWS2_CASE
    return XMA_ERR_UNSUPPORTED;
}

// One scheduler slot of the current device for one launch, cleared on `stream` in front of the launch. The
// slots go round: a launch meets a slot that an earlier launch still uses only with SCHED_SLOTS weight-gradient
// GEMMs in flight on one device at once.
static int sched_slot(cudaStream_t stream, DwSched** out) {
    static std::mutex mu;
    static DwSched* base[64] = {nullptr};
    static unsigned next[64] = {0};
    int dev = 0;
    XMA_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return XMA_ERR_UNSUPPORTED;
    DwSched* slot;
    {
        std::lock_guard<std::mutex> lock(mu);
        if (!base[dev]) {
            void* p = nullptr;
            XMA_CUDA_TRY(cudaGetSymbolAddress(&p, g_dw_sched));
            base[dev] = static_cast<DwSched*>(p);
        }
        slot = base[dev] + (next[dev]++ % SCHED_SLOTS);
    }
    XMA_CUDA_TRY(cudaMemsetAsync(slot, 0, sizeof(DwSched), stream));
    *out = slot;
    return XMA_OK;
}

template <typename T>
static int launch_dw2(const DwGemmArgs& g, const CUtensorMap& tx, const CUtensorMap& ty) {
    const uint32_t idesc = make_idesc_mn(g.dtype, true, true, 2 * BM, BN);
    const int64_t m_tiles = (g.m + 2 * BM - 1) / (2 * BM), n_tiles = (g.n + BN - 1) / BN;
    const bool dynamic = tuning().dw_dynamic && g.num_experts <= MAX_EXPERTS && pair_grid() / 2 <= SCHED_MAX_PAIRS &&
                         g.num_experts * m_tiles * n_tiles < (int64_t{1} << 31);
    if (dynamic) {
        auto kernel = dw_gemm_tc2_kernel<T, true>;
        int rc = set_smem2(kernel);
        if (rc) return rc;
        DwSched* sched = nullptr;
        rc = sched_slot(g.stream, &sched);
        if (rc) return rc;
        kernel<<<pair_grid(), block_threads(4), SMEM2_BYTES, g.stream>>>(
            tx, ty, g.counts, g.pad_offsets, g.num_experts, static_cast<int>(g.m), static_cast<int>(g.n),
            static_cast<T*>(g.dw), idesc, tune_word(), sched, g.device_status);
    } else {
        auto kernel = dw_gemm_tc2_kernel<T, false>;
        int rc = set_smem2(kernel);
        if (rc) return rc;
        kernel<<<pair_grid(), block_threads(4), SMEM2_BYTES, g.stream>>>(
            tx, ty, g.counts, g.pad_offsets, g.num_experts, static_cast<int>(g.m), static_cast<int>(g.n),
            static_cast<T*>(g.dw), idesc, tune_word(), nullptr, g.device_status);
    }
    return static_cast<int>(cudaGetLastError());
}

}  // namespace tc2

int rows_gemm_tc2(const RowsGemmArgs& g) {
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
    if (g.dtype == XMA_BF16) return tc2::rows_dispatch2<__nv_bfloat16>(g, ta, tb);
    return tc2::rows_dispatch2<__half>(g, ta, tb);
}

int dw_gemm_tc2(const DwGemmArgs& g) {
    if (!dw_gemm_tc_supported(g)) return XMA_ERR_UNSUPPORTED;
    if (g.num_experts == 0) return XMA_OK;
    CUtensorMap tx, ty;
    if (!tc::cached_map(&tx, g.dtype, g.x, g.m, g.rows_cap, g.x_stride, 64)) return XMA_ERR_TENSOR_MAP;
    if (!tc::cached_map(&ty, g.dtype, g.y, g.n, g.rows_cap, g.y_stride, 64)) return XMA_ERR_TENSOR_MAP;
    if (g.dtype == XMA_BF16) return tc2::launch_dw2<__nv_bfloat16>(g, tx, ty);
    return tc2::launch_dw2<__half>(g, tx, ty);
}

}  // namespace xma
