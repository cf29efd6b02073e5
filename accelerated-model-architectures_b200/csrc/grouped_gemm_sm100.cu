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
// timeout bit of the device status word, leaves its loops and releases tensor memory.
#include <cuda.h>

#include <cstdlib>
#include <mutex>

#include "gemm_internal.h"

namespace xma {
namespace tc {

constexpr int BM = 128;           // rows of a tile = tensor-memory lanes
constexpr int BN = 256;           // accumulator columns per tile
constexpr int BK = 64;            // reduction elements per stage (64 x 2 bytes = one 128-byte swizzle row)
constexpr int UMMA_K = 16;        // reduction elements per tcgen05.mma for 16-bit inputs
constexpr int STAGES = 4;
constexpr int MAX_EPI_WARPS = 8;  // 4 or 8 epilogue warps (block size 192 or 320): with 8, two warps share a
                                  // tensor-memory lane quarter and each takes half of the tile's columns
constexpr int THREADS = 64 + MAX_EPI_WARPS * 32;
constexpr int A_STAGE_BYTES = BM * BK * 2;  // 16 KiB
constexpr int B_STAGE_BYTES = BN * BK * 2;  // 32 KiB
constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
constexpr int TMEM_COLS = 512;
constexpr int MAX_EXPERTS = 1024;
constexpr int CHUNK_BYTES = 64 * BK * 2;  // one 64 x 64 box of an MN-major operand: 8 KiB
constexpr size_t SMEM_BYTES = 1024 /*alignment slack*/ + static_cast<size_t>(STAGES) * STAGE_BYTES +
                              (MAX_EXPERTS + 1) * sizeof(int) + 256 /*barriers*/;
constexpr unsigned long long WAIT_LIMIT_NS = 2000000000ull;

// ---- PTX wrappers ---------------------------------------------------------------------------------

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ unsigned long long globaltimer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t"
        "}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

// Bounded wait. Returns false when the CTA-wide abort flag is up or the time limit ran out
// (in which case it raises the flag).
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
    if (mbar_try_wait(bar, parity)) return true;
    const unsigned long long t0 = globaltimer_ns();
    uint32_t spins = 0;
    while (!mbar_try_wait(bar, parity)) {
        if ((++spins & 0xffu) == 0u) {
            if (*abort_flag) return false;
            if (globaltimer_ns() - t0 > WAIT_LIMIT_NS) {
                *abort_flag = 1;
                return false;
            }
        }
    }
    return true;
}

__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        :
        : "r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
        : "memory");
}

__device__ __forceinline__ void tmem_alloc(uint32_t* smem_result, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
                 "r"(cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// D[tmem] (+)= A[smem] * B[smem]^T, 128 x 256 x 16, issued by one thread.
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                         uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
        "}"
        :
        : "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}

// mbarrier arrives once every tcgen05.mma issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}

// 32 lanes x 32 consecutive 32-bit columns: thread i of the warp receives lane (base + i).
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
          "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
          "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr)
        : "memory");
}

__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// ---- descriptors ------------------------------------------------------------------------------------

// Shared-memory matrix descriptor, 128-byte swizzle, tile base 1024-byte aligned:
//   bits [0,14)  start address >> 4          bits [16,30) leading-dimension byte offset >> 4
//   bits [32,46) stride-dimension byte offset >> 4          bits [46,48) version = 1
//   bits [61,64) layout type: 2 = 128-byte swizzle
// K-major operand (reduction dimension contiguous, rows of 128 bytes): eight-row groups are 1024
// bytes apart (stride offset); the leading offset is not used by swizzled K-major layouts.
// MN-major operand (row/column index contiguous in runs of 64 elements = 128 bytes): eight
// reduction steps are 1024 bytes apart (stride offset); the next run of 64 along M/N starts one
// 64 x 64 box (8 KiB) later (leading offset).
__device__ __forceinline__ uint64_t smem_desc(uint32_t saddr, bool mn_major) {
    const uint64_t lbo = mn_major ? (CHUNK_BYTES >> 4) : 1;
    const uint64_t sbo = 1024 >> 4;
    return static_cast<uint64_t>((saddr >> 4) & 0x3fffu) | (lbo << 16) | (sbo << 32) | (1ull << 46) | (2ull << 61);
}

// Descriptor step per tcgen05.mma (16 reduction elements), in units of 16 bytes.
__device__ __forceinline__ constexpr uint32_t desc_k_step(bool mn_major) {
    return mn_major ? ((UMMA_K * 128) >> 4) : ((UMMA_K * 2) >> 4);
}

// Instruction descriptor (kind::f16): fp32 accumulate, a/b format (0 = fp16, 1 = bf16), operand
// majorness, N >> 3 at bit 17, M >> 4 at bit 24.
inline uint32_t make_idesc(int dtype, bool a_mn, bool b_mn) {
    const uint32_t fmt = (dtype == XMA_BF16) ? 1u : 0u;
    return (1u << 4) | (fmt << 7) | (fmt << 10) | ((a_mn ? 1u : 0u) << 15) | ((b_mn ? 1u : 0u) << 16) |
           (static_cast<uint32_t>(BN >> 3) << 17) | (static_cast<uint32_t>(BM >> 4) << 24);
}

// ---- epilogue helpers ----------------------------------------------------------------------------------

template <typename T>
__device__ __forceinline__ uint32_t pack2(float lo, float hi);
template <>
__device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}
template <>
__device__ __forceinline__ uint32_t pack2<__half>(float lo, float hi) {
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// Logistic function for the 16-bit epilogues: ex2.approx + rcp.approx (a few ulp in fp32, far below
// the rounding of the bf16/fp16 result it feeds).
__device__ __forceinline__ float fast_sigmoid(float x) { return __fdividef(1.0f, 1.0f + __expf(-x)); }

template <typename T>
__device__ __forceinline__ float round_to(float x) {
    return to_f32(from_f32<T>(x));
}

template <typename T>
__device__ __forceinline__ void unpack8(const uint4& q, float (&f)[8]) {
    const T* p = reinterpret_cast<const T*>(&q);
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] = to_f32(p[i]);
}

template <typename T>
__device__ __forceinline__ uint4 pack8(const float* f) {
    uint4 q;
    q.x = pack2<T>(f[0], f[1]);
    q.y = pack2<T>(f[2], f[3]);
    q.z = pack2<T>(f[4], f[5]);
    q.w = pack2<T>(f[6], f[7]);
    return q;
}

struct Shared {
    uint8_t* stage_base;  // 1024-byte aligned
    int* tile_prefix;     // [E + 1]
    uint64_t* full;       // [STAGES]
    uint64_t* empty;      // [STAGES]
    uint64_t* acc_full;   // [2]
    uint64_t* acc_empty;  // [2]
    uint32_t* tmem_ptr;
    volatile int* abort_flag;
};

__device__ __forceinline__ Shared carve_smem(uint8_t* raw) {
    Shared s;
    const uint32_t a = smem_u32(raw);
    uint8_t* base = raw + ((1024u - (a & 1023u)) & 1023u);
    s.stage_base = base;
    uint8_t* p = base + static_cast<size_t>(STAGES) * STAGE_BYTES;
    s.tile_prefix = reinterpret_cast<int*>(p);
    p += (MAX_EXPERTS + 1) * sizeof(int);
    p = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(p) + 7) & ~static_cast<uintptr_t>(7));
    s.full = reinterpret_cast<uint64_t*>(p);
    s.empty = s.full + STAGES;
    s.acc_full = s.empty + STAGES;
    s.acc_empty = s.acc_full + 2;
    s.tmem_ptr = reinterpret_cast<uint32_t*>(s.acc_empty + 2);
    s.abort_flag = reinterpret_cast<volatile int*>(s.tmem_ptr + 1);
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
// Work order: expert-major, then column tile, then row tile inside the expert, so the CTAs of one
// wave share weight tiles and the expert's activations stay in L2.
// ======================================================================================================
struct RowsWork {
    int m_tile, n_tile, e;
};

__device__ __forceinline__ RowsWork decode_rows(const int* tile_prefix, int E, int n_tiles, int64_t w) {
    // largest e with tile_prefix[e] * n_tiles <= w
    int lo = 0, hi = E;  // invariant: prefix[lo]*n_tiles <= w < prefix[hi]*n_tiles
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (static_cast<int64_t>(tile_prefix[mid]) * n_tiles <= w) lo = mid;
        else hi = mid;
    }
    RowsWork r;
    r.e = lo;
    const int64_t local = w - static_cast<int64_t>(tile_prefix[lo]) * n_tiles;
    const int mt = tile_prefix[lo + 1] - tile_prefix[lo];
    r.n_tile = static_cast<int>(local / mt);
    r.m_tile = tile_prefix[lo] + static_cast<int>(local % mt);
    return r;
}

template <typename T, int WL, int EPI>
__global__ void __launch_bounds__(THREADS, 1)
rows_gemm_tc_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                    T* __restrict__ out, int64_t out_stride, T* __restrict__ aux, int64_t aux_stride,
                    const int* __restrict__ row_map, const int* __restrict__ g_tile_prefix, int E, int kd, int n,
                    uint32_t idesc, int* __restrict__ status) {
    extern __shared__ __align__(16) uint8_t smem_raw[];
    const Shared s = carve_smem(smem_raw);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    for (int i = threadIdx.x; i <= E; i += blockDim.x) s.tile_prefix[i] = g_tile_prefix[i];
    const uint32_t tmem_base = prologue(s, warp, lane);

    constexpr bool B_MN = (WL == W_KN);
    const int half_n = n / 2;  // SwiGLU: width of the activation
    const int n_tiles = (EPI == EPI_SWIGLU) ? (half_n + 127) / 128 : (n + BN - 1) / BN;
    const int k_blocks = (kd + BK - 1) / BK;
    const int64_t total = static_cast<int64_t>(s.tile_prefix[E]) * n_tiles;

    if (warp == 0) {
        if (lane == 0) {
            uint32_t it = 0;
            for (int64_t w = blockIdx.x; w < total; w += gridDim.x) {
                const RowsWork wk = decode_rows(s.tile_prefix, E, n_tiles, w);
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
        uint32_t lt = 0;
        for (int64_t w = blockIdx.x; w < total; w += gridDim.x, ++lt) {
            const RowsWork wk = decode_rows(s.tile_prefix, E, n_tiles, w);
            const uint32_t buf = lt & 1u;
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + buf * BN;
            const int64_t r = static_cast<int64_t>(wk.m_tile) * BM + row_in_tile;

            if (EPI == EPI_PLAIN) {
                int64_t dst = r;
                if (row_map) dst = row_map[r];
                const int n0 = wk.n_tile * BN;
                if (!mbar_wait(&s.acc_full[buf], (lt >> 1) & 1u, s.abort_flag)) break;
                tc_fence_after();
#pragma unroll 1
                for (int c = part * chunks; c < (part + 1) * chunks; ++c) {
                    uint32_t v[32];
                    tmem_ld32(taddr + c * 32, v);
                    tmem_ld_wait();
                    const int col = n0 + c * 32;
                    if (dst >= 0 && col < n) {
                        T* p = out + dst * out_stride + col;
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            if (col + 8 * i < n)
                                *reinterpret_cast<uint4*>(p + 8 * i) =
                                    pack8<T>(reinterpret_cast<const float*>(&v[8 * i]));
                        }
                    }
                }
            } else if (EPI == EPI_SWIGLU) {
                const int j0 = wk.n_tile * 128;
                if (!mbar_wait(&s.acc_full[buf], (lt >> 1) & 1u, s.abort_flag)) break;
                tc_fence_after();
#pragma unroll 1
                for (int c = part * (chunks / 2); c < (part + 1) * (chunks / 2); ++c) {
                    uint32_t g[32], u[32];
                    tmem_ld32(taddr + c * 32, g);
                    tmem_ld32(taddr + 128 + c * 32, u);
                    tmem_ld_wait();
                    const int col = j0 + c * 32;
                    if (col < half_n) {
                        T* pg = aux + r * aux_stride + col;
                        T* pu = pg + half_n;
                        T* po = out + r * out_stride + col;
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            if (col + 8 * i < half_n) {
                                float gr[8], ur[8], ac[8];
#pragma unroll
                                for (int t = 0; t < 8; ++t) {
                                    gr[t] = round_to<T>(__uint_as_float(g[8 * i + t]));
                                    ur[t] = round_to<T>(__uint_as_float(u[8 * i + t]));
                                    ac[t] = ur[t] * gr[t] * fast_sigmoid(gr[t]);
                                }
                                *reinterpret_cast<uint4*>(pg + 8 * i) = pack8<T>(gr);
                                *reinterpret_cast<uint4*>(pu + 8 * i) = pack8<T>(ur);
                                *reinterpret_cast<uint4*>(po + 8 * i) = pack8<T>(ac);
                            }
                        }
                    }
                }
            } else {  // EPI_DSWIGLU: n is the activation width
                const int n0 = wk.n_tile * BN;
                const T* pg_row = aux + r * aux_stride;
                T* pd_row = out + r * out_stride;
                // gate|up of this row do not depend on the accumulator: fetch the first chunk before
                // waiting for it, and every later chunk while the previous one is being computed
                uint4 gq[2][4], uq[2][4];
                auto fetch = [&](int c, int b) {
                    const int col = n0 + c * 32;
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        if (col + 8 * i < n) {
                            gq[b][i] = *reinterpret_cast<const uint4*>(pg_row + col + 8 * i);
                            uq[b][i] = *reinterpret_cast<const uint4*>(pg_row + n + col + 8 * i);
                        }
                    }
                };
                fetch(part * chunks, 0);
                if (!mbar_wait(&s.acc_full[buf], (lt >> 1) & 1u, s.abort_flag)) break;
                tc_fence_after();
#pragma unroll
                for (int cc = 0; cc < BN / 32; ++cc) {
                    if (cc >= chunks) break;
                    const int c = part * chunks + cc;
                    if (cc + 1 < chunks) fetch(c + 1, (cc + 1) & 1);
                    uint32_t v[32];
                    tmem_ld32(taddr + c * 32, v);
                    tmem_ld_wait();
                    const int col = n0 + c * 32;
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        if (col + 8 * i < n) {
                            float gg[8], uu[8], dg[8], du[8];
                            unpack8<T>(gq[cc & 1][i], gg);
                            unpack8<T>(uq[cc & 1][i], uu);
#pragma unroll
                            for (int t = 0; t < 8; ++t) {
                                const float d = __uint_as_float(v[8 * i + t]);
                                const float sg = fast_sigmoid(gg[t]);
                                dg[t] = d * uu[t] * sg * (1.0f + gg[t] * (1.0f - sg));
                                du[t] = d * gg[t] * sg;
                            }
                            *reinterpret_cast<uint4*>(pd_row + col + 8 * i) = pack8<T>(dg);
                            *reinterpret_cast<uint4*>(pd_row + n + col + 8 * i) = pack8<T>(du);
                        }
                    }
                }
            }
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
constexpr int DW_GROUP_M = 8;

struct DwWork {
    int e, m_tile, n_tile;
};

__device__ __forceinline__ DwWork decode_dw(int64_t w, int m_tiles, int n_tiles) {
    DwWork r;
    const int64_t per_e = static_cast<int64_t>(m_tiles) * n_tiles;
    r.e = static_cast<int>(w / per_e);
    const int local = static_cast<int>(w - r.e * per_e);
    const int group_size = DW_GROUP_M * n_tiles;
    const int g = local / group_size;
    const int first_m = g * DW_GROUP_M;
    const int gm = min(DW_GROUP_M, m_tiles - first_m);
    const int in_g = local - g * group_size;
    r.m_tile = first_m + in_g % gm;
    r.n_tile = in_g / gm;
    return r;
}

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
            if (!mbar_wait(&s.acc_full[buf], (lt >> 1) & 1u, s.abort_flag)) break;
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

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    });
    return fn;
}

// Row-major 2-D tensor [outer, inner] of 16-bit elements, box [box_outer, 64], 128-byte swizzle,
// out-of-range elements read as zero.
static bool make_map(CUtensorMap* map, int dtype, const void* base, uint64_t inner, uint64_t outer,
                     uint64_t row_stride_elems, uint32_t box_outer) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    const cuuint64_t dims[2] = {inner, outer};
    const cuuint64_t strides[1] = {row_stride_elems * 2};
    const cuuint32_t box[2] = {64, box_outer};
    const cuuint32_t estr[2] = {1, 1};
    const CUtensorMapDataType dt =
        (dtype == XMA_BF16) ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    CUresult r = fn(map, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return false;
    // Drivers up to 13.1 mis-handle tensors below 128 KiB unless this descriptor bit is cleared
    // (the same adjustment CUTLASS applies after encoding).
    int drv = 0;
    if (cudaDriverGetVersion(&drv) == cudaSuccess && drv <= 13010) {
        if (outer * row_stride_elems * 2 < 131072ull) reinterpret_cast<uint64_t*>(map)[1] &= ~(1ull << 21);
    }
    return true;
}

static bool device_is_sm100() {
    static int cached = -1;
    if (cached < 0) {
        int dev = 0, major = 0;
        if (cudaGetDevice(&dev) != cudaSuccess) return false;
        if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) return false;
        cached = (major == 10) ? 1 : 0;
    }
    return cached == 1;
}

// Epilogue warps per kernel: 4 (block of 192 threads) or 8 (320). XMA_B200_EPI_WARPS=4|8 overrides
// the per-kernel default (tuning knob).
static int block_threads(int default_epi_warps) {
    static int forced = -1;
    if (forced < 0) {
        const char* e = getenv("XMA_B200_EPI_WARPS");
        forced = (e && (e[0] == '4' || e[0] == '8')) ? (e[0] - '0') : 0;
    }
    const int warps = forced ? forced : default_epi_warps;
    return 64 + 32 * warps;
}

template <typename K>
static int set_smem(K kernel) {
    return static_cast<int>(
        cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(SMEM_BYTES)));
}

template <typename T, int WL, int EPI>
static int launch_rows(const RowsGemmArgs& g, const CUtensorMap& ta, const CUtensorMap& tb) {
    auto kernel = rows_gemm_tc_kernel<T, WL, EPI>;
    int rc = set_smem(kernel);
    if (rc) return rc;
    const uint32_t idesc = make_idesc(g.dtype, false, WL == W_KN);
    kernel<<<num_sms(), block_threads(EPI == EPI_DSWIGLU ? 8 : 4), SMEM_BYTES, g.stream>>>(
        ta, tb, static_cast<T*>(g.out), g.out_stride, static_cast<T*>(g.aux), g.aux_stride, g.row_map,
        g.tile_prefix, g.num_experts, static_cast<int>(g.kd), static_cast<int>(g.n), idesc, g.device_status);
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
    const bool combo = (g.w_layout == W_NK && (g.epilogue == EPI_PLAIN || g.epilogue == EPI_SWIGLU)) ||
                       (g.w_layout == W_KN && (g.epilogue == EPI_PLAIN || g.epilogue == EPI_DSWIGLU));
    if (!combo) return false;
    if (g.epilogue != EPI_PLAIN) {
        if (!g.aux || g.aux_stride % 8 || !is_aligned16(g.aux) || g.row_map) return false;
        if (g.epilogue == EPI_SWIGLU && (g.n % 16)) return false;
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
    if (!tc::make_map(&ta, g.dtype, g.a, g.kd, rows_cap, g.a_stride, tc::BM)) return XMA_ERR_TENSOR_MAP;
    bool ok;
    if (g.w_layout == W_NK)
        ok = tc::make_map(&tb, g.dtype, g.w, g.kd, static_cast<uint64_t>(g.num_experts) * g.n, g.kd, 128);
    else
        ok = tc::make_map(&tb, g.dtype, g.w, g.n, static_cast<uint64_t>(g.num_experts) * g.kd, g.n, 64);
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
    if (!tc::make_map(&tx, g.dtype, g.x, g.m, g.rows_cap, g.x_stride, 64)) return XMA_ERR_TENSOR_MAP;
    if (!tc::make_map(&ty, g.dtype, g.y, g.n, g.rows_cap, g.y_stride, 64)) return XMA_ERR_TENSOR_MAP;
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
