// Device and host helpers shared by the tcgen05 grouped-GEMM translation units: tile constants, PTX
// wrappers (mbarrier, TMA, tcgen05), shared-memory / instruction descriptors, epilogue packing, TMA
// tensor-map creation.
#pragma once

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
// Staging of the plain epilogue when its rows go to other ranks' memory: 32 rows x 64 columns of
// 16-bit values per epilogue warp (4 warps), so that a warp store covers 128 contiguous bytes per row.
constexpr int PEER_STAGE_WARP_BYTES = 32 * 128;
constexpr int PEER_STAGE_BYTES = 4 * PEER_STAGE_WARP_BYTES;
constexpr size_t SMEM_BYTES = 1024 /*alignment slack*/ + static_cast<size_t>(STAGES) * STAGE_BYTES +
                              2 * (MAX_EXPERTS + 1) * sizeof(int) /*tile tables*/ + 256 /*barriers*/ +
                              PEER_STAGE_BYTES;
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

// How the epilogue warps wait for an accumulator: 0 = every lane polls on its own (default), 1 = one
// elected lane polls with a short sleep between polls and the warp re-converges. Measured on B200 under
// the power cap: the elected variant is 1.7 % slower on the whole layer (the sleep adds latency, the
// saved polling buys no clock). Set per translation unit before the first launch (XMA_B200_EPI_WAIT).
static __device__ int g_epi_wait_elected = 0;

__device__ __forceinline__ bool mbar_wait_epilogue(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
    if (!g_epi_wait_elected) return mbar_wait(bar, parity, abort_flag);
    int ok = 1;
    if ((threadIdx.x & 31) == 0) {
        if (!mbar_try_wait(bar, parity)) {
            const unsigned long long t0 = globaltimer_ns();
            uint32_t spins = 0;
            while (!mbar_try_wait(bar, parity)) {
                __nanosleep(64);
                if ((++spins & 0x3fu) == 0u) {
                    if (*abort_flag) { ok = 0; break; }
                    if (globaltimer_ns() - t0 > WAIT_LIMIT_NS) { *abort_flag = 1; ok = 0; break; }
                }
            }
        }
    }
    ok = __shfl_sync(0xffffffffu, ok, 0);
    __syncwarp();
    return ok != 0;
}

__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        :
        : "r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
        : "memory");
}

// Asks the TMA unit to bring one box of the tensor into L2 (no shared-memory destination, no barrier).
__device__ __forceinline__ void tma_prefetch_2d(const CUtensorMap* map, int c0, int c1) {
    asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global [%0, {%1, %2}];"
                 :
                 : "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1)
                 : "memory");
}

// Shared memory -> global through a tensor map (bulk group of the issuing thread).
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, const void* smem_src, int c0, int c1) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                 :
                 : "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(smem_src)), "r"(c0), "r"(c1)
                 : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// The issuing thread's earlier bulk stores have read their shared-memory source / have completed.
__device__ __forceinline__ void tma_store_wait_read() {
    asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}
__device__ __forceinline__ void tma_store_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
// Orders this thread's shared-memory writes before later accesses of the asynchronous (TMA) proxy.
__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// One 128-byte line into L2.
__device__ __forceinline__ void prefetch_l2(const void* p) {
    asm volatile("prefetch.global.L2 [%0];" ::"l"(p));
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
inline uint32_t make_idesc_mn(int dtype, bool a_mn, bool b_mn, int m, int n) {
    const uint32_t fmt = (dtype == XMA_BF16) ? 1u : 0u;
    return (1u << 4) | (fmt << 7) | (fmt << 10) | ((a_mn ? 1u : 0u) << 15) | ((b_mn ? 1u : 0u) << 16) |
           (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24);
}

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


// ---- epilogue of one rows-GEMM tile (shared by the 1-CTA and the 2-CTA kernels) --------------------------
// Executed by every epilogue thread: thread = one accumulator row (tensor-memory lane), `part` /
// `chunks` = which 32-column chunks of the 256 this warp handles. Waits for the accumulator itself
// (the dSwiGLU variant fetches gate|up first). `active` is CTA-uniform: false for a tile half that
// lies beyond the expert's rows (nothing is loaded or stored, the barrier protocol still runs).
// Returns false when the bounded wait gave up.
template <typename T, int EPI>
__device__ __forceinline__ bool rows_epilogue_tile(uint64_t* acc_full_bar, uint32_t parity, volatile int* abort_flag,
                                                   uint32_t taddr, int64_t r, bool active, int n_tile, int n,
                                                   int half_n, T* __restrict__ out, int64_t out_stride,
                                                   T* __restrict__ aux, int64_t aux_stride,
                                                   const int* __restrict__ row_map,
                                                   void* const* __restrict__ out_peers, int peer_world,
                                                   int64_t peer_rows_cap, int* __restrict__ status,
                                                   uint8_t* peer_stage, int part, int chunks) {
    if (!active) return mbar_wait_epilogue(acc_full_bar, parity, abort_flag);
    if (EPI == EPI_PLAIN) {
        int64_t dst = r;
        if (row_map) dst = row_map[r];
        const int n0 = n_tile * BN;
        if (!mbar_wait_epilogue(acc_full_bar, parity, abort_flag)) return false;
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
    } else if (EPI == EPI_PLAIN_PEER) {
        // Plain store whose rows go to other ranks' memory: row_map[r] = (rank << 24) | row of that rank's
        // buffer. A thread owns one row, so direct stores would be 32 pieces of 16 bytes in 32 rows per warp
        // instruction, which NVLink moves poorly. Two chunks (64 columns) are staged in shared memory
        // (16-byte pieces XOR-swizzled by row: conflict-free both ways) and stored 4 rows x 128 contiguous
        // bytes at a time; the row addresses travel between lanes by shuffle.
        // A word that names a rank outside the table or a row outside that rank's buffer is treated like a
        // negative one (nothing is stored) and raises status bit 1: a stale or corrupt word must not
        // become a store into another GPU's memory.
        int64_t dst = row_map[r];
        if (dst >= 0) {
            const int64_t owner = dst >> PEER_ROW_BITS;
            dst &= PEER_ROW_MASK;
            if (owner >= peer_world || dst >= peer_rows_cap) {
                if (status) atomicOr(status, XMA_DEV_ID_OUT_OF_RANGE);
                dst = -1;
            } else {
                out = static_cast<T*>(out_peers[owner]);
            }
        }
        const int n0 = n_tile * BN;
        if (!mbar_wait_epilogue(acc_full_bar, parity, abort_flag)) return false;
        tc_fence_after();
        if (peer_stage && (chunks & 1) == 0) {
            const int lane = threadIdx.x & 31;
            const uint64_t row_addr = (dst >= 0) ? reinterpret_cast<uint64_t>(out + dst * out_stride) : 0ull;
            const uint32_t addr_lo = static_cast<uint32_t>(row_addr), addr_hi = static_cast<uint32_t>(row_addr >> 32);
            uint4* stage = reinterpret_cast<uint4*>(peer_stage);  // [32 rows][8 pieces]
#pragma unroll 1
            for (int c = part * chunks; c < (part + 1) * chunks; c += 2) {
#pragma unroll 1
                for (int h = 0; h < 2; ++h) {
                    uint32_t v[32];
                    tmem_ld32(taddr + (c + h) * 32, v);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 4; ++i)
                        stage[lane * 8 + ((h * 4 + i) ^ (lane & 7))] =
                            pack8<T>(reinterpret_cast<const float*>(&v[8 * i]));
                }
                __syncwarp();
                const int col0 = n0 + c * 32;
                const int k = lane & 7;
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const int rr = i * 4 + (lane >> 3);
                    const uint4 x = stage[rr * 8 + (k ^ (rr & 7))];
                    const uint32_t lo = __shfl_sync(0xffffffffu, addr_lo, rr);
                    const uint32_t hi = __shfl_sync(0xffffffffu, addr_hi, rr);
                    T* p = reinterpret_cast<T*>((static_cast<uint64_t>(hi) << 32) | lo);
                    if (p && col0 + k * 8 < n) *reinterpret_cast<uint4*>(p + col0 + k * 8) = x;
                }
                __syncwarp();
            }
        } else {
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
        }
    } else if (EPI == EPI_SWIGLU) {
        const int j0 = n_tile * 128;
        if (!mbar_wait_epilogue(acc_full_bar, parity, abort_flag)) return false;
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
    } else if (EPI == EPI_SWIGLU_PACKED) {
        // gate/up interleaved along the columns (g, u, g, u, ...): one thread holds whole pairs.
        // aux[r, 0:n] = rounded contraction, out[r, 0:n/2] = activation.
        const int n0 = n_tile * BN;
        if (!mbar_wait_epilogue(acc_full_bar, parity, abort_flag)) return false;
        tc_fence_after();
#pragma unroll 1
        for (int c = part * chunks; c < (part + 1) * chunks; ++c) {
            uint32_t v[32];
            tmem_ld32(taddr + c * 32, v);
            tmem_ld_wait();
            const int col = n0 + c * 32;
            if (col < n) {
                T* pa = aux + r * aux_stride + col;
                T* po = out + r * out_stride + col / 2;
#pragma unroll
                for (int i = 0; i < 2; ++i) {  // 16 interleaved columns -> 8 outputs
                    if (col + 16 * i < n) {
                        float gu[16], ac[8];
#pragma unroll
                        for (int t = 0; t < 16; ++t) gu[t] = round_to<T>(__uint_as_float(v[16 * i + t]));
#pragma unroll
                        for (int t = 0; t < 8; ++t) ac[t] = gu[2 * t + 1] * gu[2 * t] * fast_sigmoid(gu[2 * t]);
                        *reinterpret_cast<uint4*>(pa + 16 * i) = pack8<T>(gu);
                        *reinterpret_cast<uint4*>(pa + 16 * i + 8) = pack8<T>(gu + 8);
                        *reinterpret_cast<uint4*>(po + 8 * i) = pack8<T>(ac);
                    }
                }
            }
        }
    } else if (EPI == EPI_DSWIGLU_PACKED) {
        // n = activation width; aux[r, 0:2n] holds gate/up interleaved; out[r, 0:2n] = d gate/d up interleaved
        const int n0 = n_tile * BN;
        const T* pg_row = aux + r * aux_stride;
        T* pd_row = out + r * out_stride;
        uint4 q[2][8];
        auto fetch = [&](int c, int b) {
            const int col = n0 + c * 32;
#pragma unroll
            for (int i = 0; i < 8; ++i)
                if (col + 4 * i < n) q[b][i] = *reinterpret_cast<const uint4*>(pg_row + 2 * col + 8 * i);
        };
        fetch(part * chunks, 0);
        if (!mbar_wait_epilogue(acc_full_bar, parity, abort_flag)) return false;
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
            for (int i = 0; i < 8; ++i) {  // 4 activation columns = 8 interleaved values
                if (col + 4 * i < n) {
                    float gu[8], dd[8];
                    unpack8<T>(q[cc & 1][i], gu);
#pragma unroll
                    for (int t = 0; t < 4; ++t) {
                        const float d = __uint_as_float(v[4 * i + t]);
                        const float g = gu[2 * t], u = gu[2 * t + 1];
                        const float sg = fast_sigmoid(g);
                        dd[2 * t] = d * u * sg * (1.0f + g * (1.0f - sg));
                        dd[2 * t + 1] = d * g * sg;
                    }
                    *reinterpret_cast<uint4*>(pd_row + 2 * col + 8 * i) = pack8<T>(dd);
                }
            }
        }
    } else {  // EPI_DSWIGLU: n is the activation width
        const int n0 = n_tile * BN;
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
        if (!mbar_wait_epilogue(acc_full_bar, parity, abort_flag)) return false;
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
    return true;
}

// The SwiGLU-backward epilogues read the gate|up rows of their tile from global memory; those rows are not
// in L2 (the buffer is gigabytes and was written a whole GEMM earlier). Called by every epilogue thread for
// the tile AFTER the one whose accumulator it is about to wait for, this asks for the lines that the thread
// will read then, so that they arrive while the tensor cores are still working on that tile.
template <typename T, int EPI>
__device__ __forceinline__ void prefetch_gate_up(const T* __restrict__ aux, int64_t aux_stride, int64_t r, int n_tile,
                                                 int n, int part, int chunks) {
    if (EPI != EPI_DSWIGLU && EPI != EPI_DSWIGLU_PACKED) return;
    const int col0 = n_tile * BN + part * chunks * 32;
    if (col0 >= n) return;
    const int cols = min(chunks * 32, n - col0);
    const char* row = reinterpret_cast<const char*>(aux + r * aux_stride);
    if (EPI == EPI_DSWIGLU) {
        const char* g = row + static_cast<int64_t>(col0) * sizeof(T);
        const char* u = g + static_cast<int64_t>(n) * sizeof(T);
        for (int off = 0; off < cols * static_cast<int>(sizeof(T)); off += 128) {
            prefetch_l2(g + off);
            prefetch_l2(u + off);
        }
    } else {
        const char* g = row + static_cast<int64_t>(2 * col0) * sizeof(T);
        for (int off = 0; off < 2 * cols * static_cast<int>(sizeof(T)); off += 128) prefetch_l2(g + off);
    }
}

// ---- order of the tiles inside one expert (rows GEMMs) ----------------------------------------------------
// The `local`-th work item of an expert with `mt` row tiles (or row-tile pairs) and `nt` column tiles. Row
// tiles are cut into balanced groups of at most `group`; inside a group the column tiles are swept with the
// group's row tiles innermost. CTAs take consecutive items and run in step along the reduction, so one wave
// reads about `group` row blocks and (CTAs / group) weight tiles once each from HBM and shares them through
// L2. With the row tiles of a whole expert innermost instead, a wave shares a single weight tile and every
// column tile streams the expert's rows again: for experts of 16384 rows that was 13.6 GB of DRAM reads in
// the down projection of the 8-expert configuration against 1.2 GB of operands.
__device__ __forceinline__ void raster_tile(int64_t local, int mt, int nt, int group, int& m, int& n) {
    const int ng = (mt + group - 1) / group;
    const int base = mt / ng, rem = mt - base * ng;  // the first `rem` groups hold base + 1 row tiles
    const int64_t big = static_cast<int64_t>(base + 1) * nt;
    int gl, m0;
    int64_t j;
    if (local < rem * big) {
        const int g = static_cast<int>(local / big);
        gl = base + 1;
        m0 = g * (base + 1);
        j = local - g * big;
    } else {
        const int64_t l2 = local - rem * big;
        const int64_t per = static_cast<int64_t>(base) * nt;
        const int g = static_cast<int>(l2 / per);
        gl = base;
        m0 = rem * (base + 1) + g * base;
        j = l2 - g * per;
    }
    n = static_cast<int>(j / gl);
    m = m0 + static_cast<int>(j % gl);
}

// ---- work decoding of the weight-gradient GEMM ----------------------------------------------------------
// Expert-major, then groups of DW_GROUP_M row tiles x all column tiles (row tile fastest).
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


// ---- host side ---------------------------------------------------------------------------------------

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_fn() {
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

// Row-major 2-D tensor [outer, inner] of 16-bit elements, box [box_outer, box_inner], out-of-range elements
// read as zero. box_inner = 64 elements (the GEMM operands): 128-byte swizzle; 32 elements (the staged
// SwiGLU-backward epilogue): 64-byte swizzle.
inline bool make_map(CUtensorMap* map, int dtype, const void* base, uint64_t inner, uint64_t outer,
                     uint64_t row_stride_elems, uint32_t box_outer, uint32_t box_inner = 64) {
    EncodeTiledFn fn = encode_fn();
    if (!fn || (box_inner != 64 && box_inner != 32)) return false;
    const cuuint64_t dims[2] = {inner, outer};
    const cuuint64_t strides[1] = {row_stride_elems * 2};
    const cuuint32_t box[2] = {box_inner, box_outer};
    const cuuint32_t estr[2] = {1, 1};
    const CUtensorMapDataType dt =
        (dtype == XMA_BF16) ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    CUresult r = fn(map, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    box_inner == 64 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return false;
    // Drivers up to 13.1 mis-handle tensors below 128 KiB unless this descriptor bit is cleared
    // (the same adjustment CUTLASS applies after encoding).
    int drv = 0;
    if (cudaDriverGetVersion(&drv) == cudaSuccess && drv <= 13010) {
        if (outer * row_stride_elems * 2 < 131072ull) reinterpret_cast<uint64_t*>(map)[1] &= ~(1ull << 21);
    }
    return true;
}

// Whether the CURRENT device is an sm_100 part (answer cached per device ordinal).
inline bool device_is_sm100() {
    static signed char cached[64] = {0};  // 0 = unknown, 1 = yes, -1 = no
    int dev = 0, major = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return false;
    const bool slot = dev >= 0 && dev < 64;
    if (slot && cached[dev] != 0) return cached[dev] > 0;
    if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) return false;
    if (slot) cached[dev] = (major == 10) ? 1 : -1;
    return major == 10;
}

// ---- tuning switches (one set per process, defined in gemm_api.cu) ---------------------------------------
// Packed into one kernel argument: bit 0 = the SwiGLU-backward epilogue asks for the next tile's gate|up
// rows in L2 while it waits for the accumulator; bits [8,16) = how many reduction blocks ahead of its loads
// the TMA producer issues L2 prefetches (0 = none); bit 16 / 17 = prefetch the A / B operand.
constexpr uint32_t TUNE_GU_PREFETCH = 1u;
__host__ __device__ inline uint32_t tune_prefetch_distance(uint32_t t) { return (t >> 8) & 0xffu; }
constexpr uint32_t TUNE_PREFETCH_A = 1u << 16;
constexpr uint32_t TUNE_PREFETCH_B = 1u << 17;

// Tensor-map cache: encoding a map is a driver call per operand per launch; the same (address, shape) pairs
// come back every step, so the last encodings are kept (mutex-guarded, a few dozen entries, oldest replaced).
inline bool cached_map(CUtensorMap* map, int dtype, const void* base, uint64_t inner, uint64_t outer,
                       uint64_t row_stride_elems, uint32_t box_outer, uint32_t box_inner = 64) {
    struct Key {
        const void* base;
        uint64_t inner, outer, stride;
        uint32_t box, box_inner;
        int dtype;
        bool operator==(const Key& o) const {
            return base == o.base && inner == o.inner && outer == o.outer && stride == o.stride && box == o.box &&
                   box_inner == o.box_inner && dtype == o.dtype;
        }
    };
    struct Entry {
        Key key;
        CUtensorMap map;
        bool used;
    };
    constexpr int N = 64;
    static Entry entries[N];
    static int next = 0;
    static std::mutex mu;
    const Key key{base, inner, outer, row_stride_elems, box_outer, box_inner, dtype};
    {
        std::lock_guard<std::mutex> lock(mu);
        for (int i = 0; i < N; ++i)
            if (entries[i].used && entries[i].key == key) {
                *map = entries[i].map;
                return true;
            }
    }
    if (!make_map(map, dtype, base, inner, outer, row_stride_elems, box_outer, box_inner)) return false;
    std::lock_guard<std::mutex> lock(mu);
    entries[next] = Entry{key, *map, true};
    next = (next + 1) % N;
    return true;
}

// cudaFuncAttributeMaxDynamicSharedMemorySize is a per-device property of a kernel: set it on the first launch
// of each kernel on each device only. Kernels are told apart by their address (template instances of one
// signature share a pointer TYPE, so a static per instantiation of this function would not do).
template <typename K>
inline int set_dynamic_smem_once(K kernel, size_t bytes) {
    struct Done {
        const void* fn;
        int dev;
    };
    constexpr int N = 256;
    static Done done[N];
    static int count = 0;
    static std::mutex mu;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) dev = -1;
    const void* fn = reinterpret_cast<const void*>(kernel);
    {
        std::lock_guard<std::mutex> lock(mu);
        for (int i = 0; i < count; ++i)
            if (done[i].fn == fn && done[i].dev == dev) return 0;
    }
    const int rc = static_cast<int>(
        cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(bytes)));
    if (rc == 0 && dev >= 0) {
        std::lock_guard<std::mutex> lock(mu);
        if (count < N) done[count++] = Done{fn, dev};
    }
    return rc;
}

// Copies the epilogue-wait switch from the environment into this translation unit's device variable (once;
// every translation unit that includes this header has its own copy of it).
static inline void apply_epilogue_tuning() {
    static bool done = false;
    if (done) return;
    done = true;
    const char* e = getenv("XMA_B200_EPI_WAIT");
    if (e && (e[0] == '0' || e[0] == '1')) {
        const int v = e[0] - '0';
        cudaMemcpyToSymbol(g_epi_wait_elected, &v, sizeof(int));
    }
}

// Threads per CTA: two control warps + 4 or 8 epilogue warps (per-kernel default unless the tuning switch
// forces one).
inline int block_threads(int default_epi_warps) {
    const int forced = tuning().epi_warps;
    const int warps = (forced == 4 || forced == 8) ? forced : default_epi_warps;
    return 64 + 32 * warps;
}

}  // namespace tc
}  // namespace xma
