// Routing kernels of the MoE hot path for sm_100a:
//   * continuous_count : histogram of expert ids (xma/functional/continuous_count/__init__.py:16)
//   * route_topk_softmax (+ backward): top-k over router logits and softmax over the k picked
//     values (xma/layers/moe/__init__.py:182-195, 256-262)
//   * count_sort : replaces `selected_experts.flatten().sort()` + continuous_count + cumsum
//     (xma/layers/moe/__init__.py:210-217) by a stable counting sort: per-tile histograms -> table
//     kernel -> single-pass scan over the tiles (decoupled look-back) -> stable scatter.
//
// Integer outputs are bit-exact functions of the input: counts equal bincount, the permutation is
// the stable ascending order (ties by flat index), top-k ties go to the lowest expert index.
#include "common.cuh"

#include <mutex>

namespace xma {

// ------------------------------------------------------------------------------------------------
// Histogram
// ------------------------------------------------------------------------------------------------

constexpr int HIST_THREADS = 512;
constexpr int HIST_SMEM_BYTES = 48 * 1024;

template <typename IdT, bool USE_SMEM>
__device__ __forceinline__ void hist_add(IdT id, int bins, unsigned* __restrict__ my, unsigned* __restrict__ out,
                                         bool& bad) {
    if (static_cast<unsigned long long>(id) < static_cast<unsigned long long>(bins)) {
        if (USE_SMEM) {
            atomicAdd(&my[id], 1u);
        } else {
            atomicAdd(&out[id], 1u);
        }
    } else {
        bad = true;
    }
}

// Each CTA keeps `copies` private histograms in shared memory (one per group of warps) to spread
// same-bin contention, streams its share of the ids with 128-bit loads, and adds its non-zero
// partial counts to the global counters once at the end. Ids outside [0, bins) are skipped and
// flagged in the status word.
template <typename IdT, bool USE_SMEM>
__global__ void __launch_bounds__(HIST_THREADS)
histogram_kernel(const IdT* __restrict__ ids, int64_t n, int bins, int copies, unsigned* __restrict__ out,
                 int* __restrict__ status) {
    extern __shared__ unsigned s_hist[];
    const int tid = threadIdx.x;
    unsigned* my = nullptr;
    if (USE_SMEM) {
        for (int i = tid; i < copies * bins; i += HIST_THREADS) s_hist[i] = 0u;
        __syncthreads();
        my = s_hist + ((tid >> 5) % copies) * bins;
    }

    constexpr int V = 16 / sizeof(IdT);
    bool bad = false;

    // Elements in front of the first 16-byte boundary, and behind the last full packet, go one by one.
    int64_t head = ((16 - (reinterpret_cast<uintptr_t>(ids) & 15u)) & 15u) / sizeof(IdT);
    if (head > n) head = n;
    const int64_t nvec = (n - head) / V;
    const int64_t tail_start = head + nvec * V;

    if (blockIdx.x == 0) {
        for (int64_t i = tid; i < head; i += HIST_THREADS) hist_add<IdT, USE_SMEM>(ids[i], bins, my, out, bad);
        for (int64_t i = tail_start + tid; i < n; i += HIST_THREADS)
            hist_add<IdT, USE_SMEM>(ids[i], bins, my, out, bad);
    }

    const IdT* body = ids + head;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * HIST_THREADS;
    int64_t v = static_cast<int64_t>(blockIdx.x) * HIST_THREADS + tid;
    // Two packets in flight per thread.
    for (; v + stride < nvec; v += 2 * stride) {
        Vec16<IdT> a = load16_stream(body + v * V);
        Vec16<IdT> b = load16_stream(body + (v + stride) * V);
#pragma unroll
        for (int j = 0; j < V; ++j) hist_add<IdT, USE_SMEM>(a.v[j], bins, my, out, bad);
#pragma unroll
        for (int j = 0; j < V; ++j) hist_add<IdT, USE_SMEM>(b.v[j], bins, my, out, bad);
    }
    for (; v < nvec; v += stride) {
        Vec16<IdT> a = load16_stream(body + v * V);
#pragma unroll
        for (int j = 0; j < V; ++j) hist_add<IdT, USE_SMEM>(a.v[j], bins, my, out, bad);
    }

    if (USE_SMEM) {
        __syncthreads();
        for (int b = tid; b < bins; b += HIST_THREADS) {
            unsigned s = 0;
            for (int c = 0; c < copies; ++c) s += s_hist[c * bins + b];
            if (s) atomicAdd(&out[b], s);
        }
    }
    if (bad && status) atomicOr(status, XMA_DEV_ID_OUT_OF_RANGE);
}

template <typename IdT>
static int launch_histogram(const IdT* ids, int64_t n, int bins, unsigned* out, int* status, cudaStream_t stream) {
    XMA_CUDA_TRY(cudaMemsetAsync(out, 0, sizeof(unsigned) * bins, stream));
    if (n == 0) return XMA_OK;
    constexpr int V = 16 / sizeof(IdT);
    int64_t want = ceil_div(n, static_cast<int64_t>(HIST_THREADS) * V * 2);
    int64_t cap = static_cast<int64_t>(num_sms()) * 4;
    int grid = static_cast<int>(want < 1 ? 1 : (want > cap ? cap : want));
    const int warps = HIST_THREADS / 32;
    int64_t per_copy = static_cast<int64_t>(bins) * sizeof(unsigned);
    if (per_copy <= HIST_SMEM_BYTES) {
        int copies = static_cast<int>(HIST_SMEM_BYTES / per_copy);
        if (copies > warps) copies = warps;
        size_t smem = static_cast<size_t>(copies) * per_copy;
        histogram_kernel<IdT, true><<<grid, HIST_THREADS, smem, stream>>>(ids, n, bins, copies, out, status);
    } else {
        histogram_kernel<IdT, false><<<grid, HIST_THREADS, 0, stream>>>(ids, n, bins, 1, out, status);
    }
    return static_cast<int>(cudaGetLastError());
}

// ------------------------------------------------------------------------------------------------
// Table kernel: everything the later stages need from the counts, in one tiny launch.
//   offsets_incl[e] : inclusive prefix sum (expert e owns sorted rows [offsets[e-1], offsets[e]))
//   pad_offsets[e]  : first row of expert e in the padded grouped layout (multiples of XMA_ROW_PAD)
//   tile_prefix[e]  : number of 128-row tiles in front of expert e; tile_prefix[E] = tiles in use
//   tile_expert[t]  : expert that owns padded tile t
// ------------------------------------------------------------------------------------------------
// tile_expert[t] for every tile in use and -1 in every pad row of row_src, by `nthreads` threads of which this is
// number `thread` (consecutive threads, consecutive addresses). Needs tile_prefix[0..E] from plan_kernel. The single
// plan CTA does this only when nothing is sorted afterwards; otherwise the CTAs of the scan kernel share it (one
// thread per expert walking its own tiles and pad rows, a store per 128-byte line, cost 0.3 ms at 64 Mi ids).
__device__ __forceinline__ void fill_tile_tables(int64_t thread, int64_t nthreads, const unsigned* __restrict__ counts,
                                                 int E, const int* __restrict__ tile_prefix,
                                                 int* __restrict__ tile_expert, int tile_cap,
                                                 int* __restrict__ row_src) {
    const int total = tile_prefix[E];
    for (int64_t t = thread; t < total; t += nthreads) {
        int lo = 0, hi = E;  // largest e with tile_prefix[e] <= t
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (tile_prefix[mid] <= t) lo = mid;
            else hi = mid;
        }
        tile_expert[t] = lo;
    }
    if (!row_src) return;
    const int64_t rows_cap = static_cast<int64_t>(tile_cap) * XMA_ROW_PAD;
    for (int64_t i = thread; i < static_cast<int64_t>(E) * XMA_ROW_PAD; i += nthreads) {  // pad rows of each expert
        const int e = static_cast<int>(i / XMA_ROW_PAD);
        const int t1 = min(tile_prefix[e + 1], total);
        const int64_t r = static_cast<int64_t>(tile_prefix[e]) * XMA_ROW_PAD + counts[e] + (i % XMA_ROW_PAD);
        if (r < static_cast<int64_t>(t1) * XMA_ROW_PAD && r < rows_cap) row_src[r] = -1;
    }
    // allocated rows behind the last expert's block
    for (int64_t r = static_cast<int64_t>(total) * XMA_ROW_PAD + thread; r < rows_cap; r += nthreads) row_src[r] = -1;
}

__global__ void plan_kernel(const unsigned* __restrict__ counts, int E, int* __restrict__ offsets_incl,
                            int* __restrict__ pad_offsets, int* __restrict__ tile_prefix,
                            int* __restrict__ tile_expert, int tile_cap, int* __restrict__ row_src,
                            int fill_tables, int* __restrict__ status) {
    __shared__ int s_cnt[1024];  // E <= 1024 (checked by the callers)
    // counts are read in parallel (one dependent global load per expert in a serial loop cost ~0.3 us each)
    for (int e = threadIdx.x; e < E; e += blockDim.x) s_cnt[e] = static_cast<int>(counts[e]);
    __syncthreads();
    if (threadIdx.x == 0) {
        int run = 0, pad = 0, tiles = 0;
        for (int e = 0; e < E; ++e) {
            const int c = s_cnt[e];
            run += c;
            offsets_incl[e] = run;
            pad_offsets[e] = pad;
            tile_prefix[e] = tiles;
            int t = (c + XMA_ROW_PAD - 1) / XMA_ROW_PAD;
            tiles += t;
            pad += t * XMA_ROW_PAD;
        }
        pad_offsets[E] = pad;
        if (tiles > tile_cap) {  // cannot happen when the caller sized the tables from n and E
            if (status) atomicOr(status, XMA_DEV_BAD_TILE);
            tiles = tile_cap;
        }
        tile_prefix[E] = tiles;
        __threadfence_block();
    }
    __syncthreads();
    if (fill_tables)
        fill_tile_tables(threadIdx.x, blockDim.x, counts, E, tile_prefix, tile_expert, tile_cap, row_src);
}

// ------------------------------------------------------------------------------------------------
// Stable counting sort: per-tile histograms -> scan over the tiles (decoupled look-back) -> scatter
// ------------------------------------------------------------------------------------------------
// The ids are cut into tiles of SORT_TILE. Pass 1 counts every bin per tile (and the global counts); the
// exclusive scan of those counts down the tiles, bin by bin, tells each tile where its share of a bin starts;
// pass 2 ranks the ids of a tile and writes them there. The scan is a single pass with a decoupled look-back
// between chunks of SCAN_TILES tiles. The look-back sits here, on 4 bytes per tile and bin, and not inside
// pass 2 (where the first version had it, one status word per tile and bin): a look-back front advances a
// fixed number of status words per round trip to L2, so with one word per 8192-id tile the whole 64 Mi-id
// sort was bounded by about 500 such round trips per bin chain (1 ms) whatever the occupancy.
constexpr int SORT_THREADS = 512;
constexpr int SORT_WARPS = SORT_THREADS / 32;
constexpr int SORT_ITEMS = 16;
constexpr int SORT_TILE = SORT_THREADS * SORT_ITEMS;  // 8192 ids per CTA
constexpr int SORT_MAX_BINS = 1024;
constexpr int SCAN_TILES = 64;    // tiles per chunk of the scan
constexpr int SCAN_THREADS = 256;
constexpr int LB_BATCH = 8;       // predecessors fetched per look-back round

// Look-back status word: [63:62] state, [31:0] value. One 64-bit store/load moves both at once,
// so no fence is needed between flag and payload.
constexpr unsigned long long LB_AGGREGATE = 1ull << 62;
constexpr unsigned long long LB_PREFIX = 2ull << 62;
constexpr unsigned long long LB_STATE_MASK = 3ull << 62;
constexpr unsigned LB_MAX_POLLS = 1u << 22;  // bounded wait; on expiry the status word gets the timeout bit

// Scratch of one count_sort call (the caller's memory, zeroed by the call before use):
//   [0, 256)            ticket counter of the scan kernel
//   tile_counts         [tiles][E] u32   per-tile counts, turned into exclusive prefixes inside the chunk
//   chunk_base          [chunks][E] u32  sorted position of the chunk's first id of the bin
//   lb                  [chunks][E] u64  look-back status words of the scan
struct SortScratch {
    unsigned* ticket;
    unsigned* tile_counts;
    unsigned* chunk_base;
    unsigned long long* lb;
    size_t bytes;
};

__host__ __device__ inline SortScratch sort_scratch_layout(unsigned char* base, int64_t n, int E) {
    int64_t tiles = (n + SORT_TILE - 1) / SORT_TILE;
    if (tiles < 1) tiles = 1;
    const int64_t chunks = (tiles + SCAN_TILES - 1) / SCAN_TILES;
    SortScratch s;
    size_t off = 256;
    s.ticket = reinterpret_cast<unsigned*>(base);
    s.tile_counts = reinterpret_cast<unsigned*>(base + off);
    off += static_cast<size_t>(tiles) * E * sizeof(unsigned);
    s.chunk_base = reinterpret_cast<unsigned*>(base + off);
    off += static_cast<size_t>(chunks) * E * sizeof(unsigned);
    off = (off + 7) & ~static_cast<size_t>(7);
    s.lb = reinterpret_cast<unsigned long long*>(base + off);
    off += static_cast<size_t>(chunks) * E * sizeof(unsigned long long);
    s.bytes = off;
    return s;
}

__host__ __device__ inline size_t sort_scratch_bytes(int64_t n, int E) {
    return sort_scratch_layout(nullptr, n, E).bytes;
}

// Pass 1. Each CTA takes whole tiles: counts them in `copies` shared-memory histograms (one per group of
// warps, which spreads same-bin contention: the MoE layer feeds nearly sorted ids), writes the tile's counts
// and keeps a running total per bin that goes to the global counters once at the end.
template <typename IdT>
__global__ void __launch_bounds__(SORT_THREADS)
tile_histogram_kernel(const IdT* __restrict__ ids, int64_t n, int E, int copies, unsigned* __restrict__ tile_counts,
                      unsigned* __restrict__ counts, int* __restrict__ status) {
    extern __shared__ unsigned s_hist[];  // [copies][E] + totals [E]
    unsigned* s_total = s_hist + copies * E;
    const int tid = threadIdx.x;
    for (int i = tid; i < (copies + 1) * E; i += SORT_THREADS) s_hist[i] = 0u;
    __syncthreads();
    unsigned* my = s_hist + ((tid >> 5) % copies) * E;
    const int64_t tiles = (n + SORT_TILE - 1) / SORT_TILE;
    constexpr int V = 16 / sizeof(IdT);
    const bool aligned = (reinterpret_cast<uintptr_t>(ids) & 15u) == 0;
    bool bad = false;
    for (int64_t tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
        const int64_t base = tile * SORT_TILE;
        const int cnt = static_cast<int>((n - base) < SORT_TILE ? (n - base) : SORT_TILE);
        if (aligned && cnt == SORT_TILE) {
            Vec16<IdT> q[SORT_ITEMS / V];
#pragma unroll
            for (int j = 0; j < SORT_ITEMS / V; ++j) q[j] = load16_stream(ids + base + (j * SORT_THREADS + tid) * V);
#pragma unroll
            for (int j = 0; j < SORT_ITEMS / V; ++j)
#pragma unroll
                for (int i = 0; i < V; ++i) hist_add<IdT, true>(q[j].v[i], E, my, nullptr, bad);
        } else {
            for (int i = tid; i < cnt; i += SORT_THREADS) hist_add<IdT, true>(ids[base + i], E, my, nullptr, bad);
        }
        __syncthreads();
        for (int b = tid; b < E; b += SORT_THREADS) {
            unsigned sum = 0;
            for (int c = 0; c < copies; ++c) {
                sum += s_hist[c * E + b];
                s_hist[c * E + b] = 0u;
            }
            tile_counts[tile * E + b] = sum;
            s_total[b] += sum;
        }
        __syncthreads();
    }
    for (int b = tid; b < E; b += SORT_THREADS)
        if (s_total[b]) atomicAdd(&counts[b], s_total[b]);
    if (bad && status) atomicOr(status, XMA_DEV_ID_OUT_OF_RANGE);
}

// Scan of one chunk of tiles, bin `b`: tile_counts[t][b] becomes the number of ids of bin b in the chunk's
// earlier tiles; returns the chunk's total. Eight independent loads at a time.
__device__ __forceinline__ unsigned scan_chunk_bin(unsigned* __restrict__ tile_counts, int64_t t0, int64_t t1, int E,
                                                   int b) {
    unsigned run = 0;
    for (int64_t t = t0; t < t1; t += 8) {
        unsigned v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = (t + j < t1) ? tile_counts[(t + j) * E + b] : 0u;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            if (t + j < t1) tile_counts[(t + j) * E + b] = run;
            run += v[j];
        }
    }
    return run;
}

// Scan over the tiles, one chunk of SCAN_TILES tiles per CTA, chunk ids handed out by an atomic ticket (so a
// waiting chunk only waits on chunks that are resident). Per bin: scan the chunk, publish its total, look back
// over the earlier chunks (LB_BATCH status words per round, independent loads) until one that already knows
// its inclusive prefix, publish the own inclusive prefix. chunk_base = bin's first sorted position + prefix.
// The wait is bounded: after LB_MAX_POLLS empty rounds the chunk sets status bit 2 and goes on with prefix 0.
__global__ void __launch_bounds__(SCAN_THREADS)
tile_scan_kernel(SortScratch sc, int64_t tiles, int E, const int* __restrict__ offsets_incl,
                 const unsigned* __restrict__ counts, const int* __restrict__ tile_prefix,
                 int* __restrict__ tile_expert, int tile_cap, int* __restrict__ row_src, int* __restrict__ status) {
    __shared__ unsigned s_chunk;
    if (threadIdx.x == 0) s_chunk = atomicAdd(sc.ticket, 1u);
    __syncthreads();
    const int64_t chunk = s_chunk;
    const int64_t t0 = chunk * SCAN_TILES;
    if (t0 >= tiles) return;
    const int64_t t1 = (t0 + SCAN_TILES < tiles) ? t0 + SCAN_TILES : tiles;
    for (int b = threadIdx.x; b < E; b += SCAN_THREADS) {
        const unsigned run = scan_chunk_bin(sc.tile_counts, t0, t1, E, b);
        unsigned long long* mine = sc.lb + static_cast<size_t>(chunk) * E + b;
        unsigned excl = 0;
        if (chunk == 0) {
            atomicExch(mine, LB_PREFIX | run);
        } else {
            atomicExch(mine, LB_AGGREGATE | run);
            int64_t prev = chunk - 1;
            unsigned polls = 0;
            bool gave_up = false, done = false;
            while (!done) {
                unsigned long long v[LB_BATCH];
#pragma unroll
                for (int j = 0; j < LB_BATCH; ++j) {
                    const int64_t t = prev - j;
                    unsigned long long word = LB_PREFIX;  // beyond chunk 0: an empty prefix
                    if (t >= 0)
                        word = *reinterpret_cast<volatile unsigned long long*>(sc.lb + static_cast<size_t>(t) * E + b);
                    v[j] = word;
                }
                int used = 0;
#pragma unroll
                for (int j = 0; j < LB_BATCH; ++j) {
                    if (done || used < j) continue;  // stop at the first unpublished entry
                    const unsigned long long st = v[j] & LB_STATE_MASK;
                    if (st == 0ull) continue;
                    excl += static_cast<unsigned>(v[j] & 0xffffffffull);
                    used = j + 1;
                    if (st == LB_PREFIX) done = true;
                }
                prev -= used;
                if (!done && used < LB_BATCH) {  // ran into a chunk that has not published yet
                    if (++polls > LB_MAX_POLLS) {
                        gave_up = true;
                        break;
                    }
                    if (used == 0) __nanosleep(32);
                }
            }
            if (gave_up) {
                if (status) atomicOr(status, XMA_DEV_WAIT_TIMEOUT);
                excl = 0;
            }
            atomicExch(mine, LB_PREFIX | static_cast<unsigned long long>(excl + run));
        }
        const unsigned gbase = (b == 0) ? 0u : static_cast<unsigned>(offsets_incl[b - 1]);
        sc.chunk_base[static_cast<size_t>(chunk) * E + b] = gbase + excl;
    }
    // the tile -> expert table and the pad rows of row_src, shared by all CTAs of this launch
    fill_tile_tables(static_cast<int64_t>(blockIdx.x) * SCAN_THREADS + threadIdx.x,
                     static_cast<int64_t>(gridDim.x) * SCAN_THREADS, counts, E, tile_prefix, tile_expert, tile_cap,
                     row_src);
}

// Pass 2, one tile of SORT_TILE ids per CTA: the tile is sorted by bin inside the CTA, stably, by a
// least-significant-digit radix sort with 4-bit digits (two passes for up to 256 bins, three up to 1024), and
// then leaves as runs of consecutive addresses (scattering straight from registers would touch one 32-byte
// sector per id). Ranking is the counter scheme of block radix sorts: thread t holds 16 consecutive elements of
// the current sequence and counts its digits in its own byte counters cnt[digit][t]; the exclusive prefix of all
// counters in (digit, thread) order is the position of a thread's first element of a digit, the count at the
// moment an element was met its offset behind that - about 20 warp instructions per 32 ids and pass, where
// the first version (one warp vote per bit of the bin index to find the lanes with equal bins, then per-warp
// counters) spent about 200 per 32 ids and was bound by instruction issue at 0.2 of the HBM roof.
// No CTA waits for another: the tile's base in every bin comes from the scanned tables.
constexpr int RADIX_BITS = 4;
constexpr int RADIX = 1 << RADIX_BITS;
constexpr unsigned SORT_INVALID = 0xffffffffu;

__host__ __device__ inline size_t sort_smem_bytes(int E) {
    // items[TILE] u32, cnt[RADIX][THREADS] u8, pref[RADIX][THREADS] u16, first[E] u32, dst_base[E] i32,
    // pad_delta[E] i32, scan scratch
    size_t b = static_cast<size_t>(SORT_TILE) * sizeof(unsigned);
    b += static_cast<size_t>(RADIX) * SORT_THREADS * (sizeof(unsigned char) + sizeof(unsigned short));
    b += 3 * static_cast<size_t>(E) * sizeof(int);
    b += 64 * sizeof(unsigned);
    return (b + 15) & ~static_cast<size_t>(15);
}

template <typename IdT>
__global__ void __launch_bounds__(SORT_THREADS, 3)
sort_scatter_kernel(const IdT* __restrict__ ids, int64_t n, int E, int passes, const int* __restrict__ offsets_incl,
                    const int* __restrict__ pad_offsets, int* __restrict__ sorted_expert,
                    int* __restrict__ sorted_scattered, int* __restrict__ row_src, int* __restrict__ row_dst,
                    SortScratch sc, int* __restrict__ status) {
    extern __shared__ __align__(16) unsigned char s_raw[];
    unsigned* s_items = reinterpret_cast<unsigned*>(s_raw);                                   // [TILE] (i << 16) | bin
    unsigned char* s_cnt = reinterpret_cast<unsigned char*>(s_items + SORT_TILE);             // [RADIX][THREADS]
    unsigned short* s_pref = reinterpret_cast<unsigned short*>(s_cnt + RADIX * SORT_THREADS);  // [RADIX][THREADS]
    unsigned* s_first = reinterpret_cast<unsigned*>(s_pref + RADIX * SORT_THREADS);           // [E]
    int* s_dst_base = reinterpret_cast<int*>(s_first + E);                                    // [E]
    int* s_pad_delta = s_dst_base + E;                                                        // [E]
    unsigned* s_scan = reinterpret_cast<unsigned*>(s_pad_delta + E);                          // [64]
    unsigned short* s_inv = reinterpret_cast<unsigned short*>(s_cnt);  // [TILE], after the passes: position of id i

    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;
    const int64_t tile = blockIdx.x;
    const int64_t base = tile * SORT_TILE;
    if (base >= n) return;  // uniform for the CTA
    const int cnt = static_cast<int>((n - base) < SORT_TILE ? (n - base) : SORT_TILE);

    // what the output step needs from global memory, asked for now so that it arrives during the sort
    // (E <= 1024 bins over 512 threads: two bins per thread)
    constexpr int BINS_PER_THREAD = SORT_MAX_BINS / SORT_THREADS;
    unsigned pre_first[BINS_PER_THREAD];
    int pre_delta[BINS_PER_THREAD];
    {
        const unsigned* tile_excl = sc.tile_counts + static_cast<size_t>(tile) * E;
        const unsigned* chunk_base = sc.chunk_base + static_cast<size_t>(tile / SCAN_TILES) * E;
#pragma unroll
        for (int j = 0; j < BINS_PER_THREAD; ++j) {
            const int b = tid + j * SORT_THREADS;
            if (b < E) {
                pre_first[j] = chunk_base[b] + tile_excl[b];  // sorted position of the tile's first id of bin b
                const int gbase = (b == 0) ? 0 : offsets_incl[b - 1];
                pre_delta[j] = pad_offsets[b] - gbase;        // padded row - sorted row
            }
        }
    }

    // 1. load: thread t takes the 16 consecutive ids [16 t, 16 t + 16) of the tile
    unsigned item[SORT_ITEMS];
    bool bad = false;
    {
        constexpr int V = 16 / sizeof(IdT);
        const IdT* src = ids + base + tid * SORT_ITEMS;
        IdT raw[SORT_ITEMS];
        if (cnt == SORT_TILE && (reinterpret_cast<uintptr_t>(ids) & 15u) == 0) {
#pragma unroll
            for (int j = 0; j < SORT_ITEMS / V; ++j) {
                const Vec16<IdT> q = load16_stream(src + j * V);
#pragma unroll
                for (int i = 0; i < V; ++i) raw[j * V + i] = q.v[i];
            }
        } else {
#pragma unroll
            for (int k = 0; k < SORT_ITEMS; ++k) raw[k] = (tid * SORT_ITEMS + k < cnt) ? src[k] : static_cast<IdT>(0);
        }
#pragma unroll
        for (int k = 0; k < SORT_ITEMS; ++k) {
            const int i = tid * SORT_ITEMS + k;
            unsigned w = SORT_INVALID;
            if (i < cnt) {
                if (static_cast<unsigned long long>(raw[k]) < static_cast<unsigned long long>(E)) {
                    w = (static_cast<unsigned>(i) << 16) | static_cast<unsigned>(raw[k]);
                } else {
                    bad = true;
                    if (row_dst) row_dst[base + i] = -1;  // a dropped id has no grouped row
                }
            }
            item[k] = w;
        }
    }

    // 2. stable radix passes, least significant digit first
    unsigned n_valid = 0;
    for (int pass = 0; pass < passes; ++pass) {
        const int shift = pass * RADIX_BITS;
        // count in registers: sixteen 8-bit counters in two 64-bit words (a thread holds at most 16 elements);
        // the value before the increment = how many elements of this digit the thread has met before. (Counting
        // straight in the shared byte counters made every element wait for the read-modify-write of the one
        // before it: the pass was bound by shared-memory latency.)
        unsigned long long c_lo = 0ull, c_hi = 0ull;  // digits 0-7, 8-15
        unsigned long long met = 0ull;                // 16 x 4 bits
#pragma unroll
        for (int k = 0; k < SORT_ITEMS; ++k) {
            if (item[k] != SORT_INVALID) {
                const unsigned d = (item[k] >> shift) & (RADIX - 1);
                const unsigned sh = (d & 7u) << 3;
                const bool high = (d & 8u) != 0u;
                const unsigned long long word = high ? c_hi : c_lo;
                const unsigned old = static_cast<unsigned>(word >> sh) & 0xffu;
                const unsigned long long inc = 1ull << sh;
                c_hi += high ? inc : 0ull;
                c_lo += high ? 0ull : inc;
                met |= static_cast<unsigned long long>(old) << (4 * k);
            }
        }
        // every thread writes all sixteen of its counters cnt[digit][t]: nothing to zero beforehand
#pragma unroll
        for (int d = 0; d < RADIX; ++d) {
            const unsigned long long word = (d & 8) ? c_hi : c_lo;
            s_cnt[d * SORT_THREADS + tid] = static_cast<unsigned char>(word >> ((d & 7) << 3));
        }
        __syncthreads();
        // scan of all counters in (digit, thread) order: thread t owns the 16 counters [16 t, 16 t + 16)
        {
            const uint4 q = reinterpret_cast<const uint4*>(s_cnt)[tid];
            const unsigned words[4] = {q.x, q.y, q.z, q.w};
            unsigned run[16];
            unsigned total = 0;
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                run[j] = total;
                total += (words[j >> 2] >> (8 * (j & 3))) & 0xffu;
            }
            unsigned incl = total;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const unsigned t = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl += t;
            }
            if (lane == 31) s_scan[warp] = incl;
            __syncthreads();
            unsigned wsum = (lane < SORT_WARPS) ? s_scan[lane] : 0u;
            unsigned winc = wsum;
#pragma unroll
            for (int o = 1; o < SORT_WARPS; o <<= 1) {
                const unsigned t = __shfl_up_sync(0xffffffffu, winc, o);
                if (lane >= o) winc += t;
            }
            const unsigned before_warp = __shfl_sync(0xffffffffu, winc - wsum, warp);
            n_valid = __shfl_sync(0xffffffffu, winc, SORT_WARPS - 1);
            const unsigned tbase = before_warp + incl - total;
            uint4 lo, hi;
            lo.x = (tbase + run[0]) | ((tbase + run[1]) << 16);
            lo.y = (tbase + run[2]) | ((tbase + run[3]) << 16);
            lo.z = (tbase + run[4]) | ((tbase + run[5]) << 16);
            lo.w = (tbase + run[6]) | ((tbase + run[7]) << 16);
            hi.x = (tbase + run[8]) | ((tbase + run[9]) << 16);
            hi.y = (tbase + run[10]) | ((tbase + run[11]) << 16);
            hi.z = (tbase + run[12]) | ((tbase + run[13]) << 16);
            hi.w = (tbase + run[14]) | ((tbase + run[15]) << 16);
            reinterpret_cast<uint4*>(s_pref)[2 * tid] = lo;
            reinterpret_cast<uint4*>(s_pref)[2 * tid + 1] = hi;
        }
        __syncthreads();
        // rank and move: position = prefix of (digit, thread) + elements of the digit met before in the thread
#pragma unroll
        for (int k = 0; k < SORT_ITEMS; ++k) {
            if (item[k] != SORT_INVALID) {
                const unsigned d = (item[k] >> shift) & (RADIX - 1);
                const unsigned pos = s_pref[d * SORT_THREADS + tid] + (static_cast<unsigned>(met >> (4 * k)) & 15u);
                s_items[pos] = item[k];
            }
        }
        __syncthreads();
        if (pass + 1 < passes) {  // next pass: the thread takes 16 consecutive elements of the new sequence
            const uint4* p = reinterpret_cast<const uint4*>(s_items + tid * SORT_ITEMS);
#pragma unroll
            for (int j = 0; j < SORT_ITEMS / 4; ++j) {
                const uint4 q = p[j];
                const unsigned w4[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const unsigned pos = tid * SORT_ITEMS + j * 4 + i;
                    item[j * 4 + i] = (pos < n_valid) ? w4[i] : SORT_INVALID;
                }
            }
            // (the barrier behind the next pass's counter reset orders these reads before its writes to s_items)
        }
    }

    // 3. tables of the output step; s_items[0, n_valid) is the tile sorted by bin
#pragma unroll
    for (int j = 0; j < BINS_PER_THREAD; ++j) {
        const int b = tid + j * SORT_THREADS;
        if (b < E) {
            s_first[b] = pre_first[j];
            s_pad_delta[b] = pre_delta[j];
        }
    }
    if (row_dst) {  // 0xffff = "id was dropped"
        const uint4 ones = make_uint4(0xffffffffu, 0xffffffffu, 0xffffffffu, 0xffffffffu);
        reinterpret_cast<uint4*>(s_inv)[2 * tid] = ones;
        reinterpret_cast<uint4*>(s_inv)[2 * tid + 1] = ones;
    }
    __syncthreads();
    const int valid = static_cast<int>(n_valid);
    // where a bin's run starts in the tile: dst_base = (first sorted position of the bin for this tile) - start
    for (int j = tid; j < valid; j += SORT_THREADS) {
        const unsigned b = s_items[j] & 0xffffu;
        if (j == 0 || (s_items[j - 1] & 0xffffu) != b) s_dst_base[b] = static_cast<int>(s_first[b]) - j;
    }
    __syncthreads();

    // 4. each bin's run goes out as consecutive addresses
    for (int j = tid; j < valid; j += SORT_THREADS) {
        const unsigned word = s_items[j];
        const unsigned b = word & 0xffffu;
        const unsigned i = word >> 16;
        const int f = static_cast<int>(base) + static_cast<int>(i);
        const int g = s_dst_base[b] + j;
        sorted_scattered[g] = f;
        sorted_expert[g] = static_cast<int>(b);
        if (row_src) row_src[g + s_pad_delta[b]] = f;
        if (row_dst) s_inv[i] = static_cast<unsigned short>(j);
    }
    if (row_dst) {  // the inverse map leaves in the order of the ids
        __syncthreads();
        for (int i = tid; i < cnt; i += SORT_THREADS) {
            const unsigned j = s_inv[i];
            if (j != 0xffffu) {
                const unsigned b = s_items[j] & 0xffffu;
                row_dst[base + i] = s_dst_base[b] + static_cast<int>(j) + s_pad_delta[b];
            }
        }
    }
    if (bad && status) atomicOr(status, XMA_DEV_ID_OUT_OF_RANGE);
}

// ------------------------------------------------------------------------------------------------
// top-k + softmax over the k selected logits
// ------------------------------------------------------------------------------------------------

// Total order used for the selection: NaN above everything (as torch.topk), then larger value,
// then lower expert index.
__device__ __forceinline__ bool cand_better(float a, int ai, float b, int bi) {
    const bool an = (a != a), bn = (b != b);
    if (an != bn) return an;
    if (!an && a != b) return a > b;
    return ai < bi;
}

constexpr int TOPK_WARPS = 8;

template <typename T, int NV>
__global__ void __launch_bounds__(TOPK_WARPS * 32)
topk_softmax_kernel(const T* __restrict__ logits, int64_t logits_stride, int64_t tokens, int E, int K,
                    T* __restrict__ weights, int* __restrict__ selected32, long long* __restrict__ selected64) {
    const int lane = threadIdx.x & 31;
    const int64_t row = static_cast<int64_t>(blockIdx.x) * TOPK_WARPS + (threadIdx.x >> 5);
    if (row >= tokens) return;
    const T* src = logits + row * logits_stride;

    float v[NV];
#pragma unroll
    for (int j = 0; j < NV; ++j) {
        int e = j * 32 + lane;
        v[j] = (e < E) ? to_f32(src[e]) : 0.0f;
    }
    unsigned taken = 0u;
#pragma unroll
    for (int j = 0; j < NV; ++j)
        if (j * 32 + lane >= E) taken |= (1u << j);

    float sel_v = 0.0f;
    int sel_i = 0;
    for (int k = 0; k < K; ++k) {
        float bv = 0.0f;
        int bi = 0x7fffffff;  // "no candidate"
#pragma unroll
        for (int j = 0; j < NV; ++j) {
            if (!((taken >> j) & 1u)) {
                int e = j * 32 + lane;
                if (bi == 0x7fffffff || cand_better(v[j], e, bv, bi)) {
                    bv = v[j];
                    bi = e;
                }
            }
        }
#pragma unroll
        for (int o = 16; o >= 1; o >>= 1) {
            float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (oi != 0x7fffffff && (bi == 0x7fffffff || cand_better(ov, oi, bv, bi))) {
                bv = ov;
                bi = oi;
            }
        }
        if ((bi & 31) == lane) taken |= (1u << (bi >> 5));
        if (lane == k) {
            sel_v = bv;
            sel_i = bi;
        }
    }

    // softmax over the K selected values, fp32
    const float vmax = __shfl_sync(0xffffffffu, sel_v, 0);
    float p = (lane < K) ? expf(sel_v - vmax) : 0.0f;
    float s = p;
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (lane < K) {
        weights[row * K + lane] = from_f32<T>(p / s);
        if (selected32) selected32[row * K + lane] = sel_i;
        if (selected64) selected64[row * K + lane] = sel_i;
    }
}

// d_logits[t, e] = w_k (dw_k - sum_j w_j dw_j) where e is the k-th selected expert of token t, else 0.
// w is recomputed in fp32 from the logits exactly as the forward did.
template <typename T, int NV>
__global__ void __launch_bounds__(TOPK_WARPS * 32)
topk_softmax_bwd_kernel(const T* __restrict__ logits, int64_t logits_stride, const int* __restrict__ selected,
                        const T* __restrict__ d_weights, int64_t tokens, int E, int K, T* __restrict__ d_logits) {
    const int lane = threadIdx.x & 31;
    const int64_t row = static_cast<int64_t>(blockIdx.x) * TOPK_WARPS + (threadIdx.x >> 5);
    if (row >= tokens) return;

    int sel = -1;
    float val = 0.0f, dw = 0.0f;
    if (lane < K) {
        sel = selected[row * K + lane];
        val = to_f32(logits[row * logits_stride + sel]);
        dw = to_f32(d_weights[row * K + lane]);
    }
    const float vmax = __shfl_sync(0xffffffffu, val, 0);
    float p = (lane < K) ? expf(val - vmax) : 0.0f;
    float s = p;
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    const float w = p / s;
    float dot = w * dw;
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
    const float dv = w * (dw - dot);

    float out[NV];
#pragma unroll
    for (int j = 0; j < NV; ++j) out[j] = 0.0f;
    for (int k = 0; k < K; ++k) {
        const int sk = __shfl_sync(0xffffffffu, sel, k);
        const float gk = __shfl_sync(0xffffffffu, dv, k);
#pragma unroll
        for (int j = 0; j < NV; ++j)
            if (sk == j * 32 + lane) out[j] = gk;
    }
    T* dst = d_logits + row * static_cast<int64_t>(E);
#pragma unroll
    for (int j = 0; j < NV; ++j) {
        int e = j * 32 + lane;
        if (e < E) dst[e] = from_f32<T>(out[j]);
    }
}

template <typename T>
static int launch_topk(const void* logits, int64_t stride, int64_t tokens, int E, int K, void* weights, int* sel32,
                       long long* sel64, cudaStream_t stream) {
    if (tokens == 0) return XMA_OK;
    const int64_t grid64 = ceil_div(tokens, TOPK_WARPS);
    if (grid64 > 0x7fffffff) return XMA_ERR_TOO_LARGE;
    const int grid = static_cast<int>(grid64);
    const T* l = static_cast<const T*>(logits);
    T* w = static_cast<T*>(weights);
#define XMA_TOPK_CASE(NV)                                                                                   \
    topk_softmax_kernel<T, NV><<<grid, TOPK_WARPS * 32, 0, stream>>>(l, stride, tokens, E, K, w, sel32, sel64)
    if (E <= 32) XMA_TOPK_CASE(1);
    else if (E <= 64) XMA_TOPK_CASE(2);
    else if (E <= 128) XMA_TOPK_CASE(4);
    else if (E <= 256) XMA_TOPK_CASE(8);
    else if (E <= 512) XMA_TOPK_CASE(16);
    else XMA_TOPK_CASE(32);
#undef XMA_TOPK_CASE
    return static_cast<int>(cudaGetLastError());
}

template <typename T>
static int launch_topk_bwd(const void* logits, int64_t stride, const int* selected, const void* d_weights,
                           int64_t tokens, int E, int K, void* d_logits, cudaStream_t stream) {
    if (tokens == 0) return XMA_OK;
    const int64_t grid64 = ceil_div(tokens, TOPK_WARPS);
    if (grid64 > 0x7fffffff) return XMA_ERR_TOO_LARGE;
    const int grid = static_cast<int>(grid64);
    const T* l = static_cast<const T*>(logits);
    const T* dw = static_cast<const T*>(d_weights);
    T* dl = static_cast<T*>(d_logits);
#define XMA_TOPKB_CASE(NV)                                                                                    \
    topk_softmax_bwd_kernel<T, NV><<<grid, TOPK_WARPS * 32, 0, stream>>>(l, stride, selected, dw, tokens, E, K, dl)
    if (E <= 32) XMA_TOPKB_CASE(1);
    else if (E <= 64) XMA_TOPKB_CASE(2);
    else if (E <= 128) XMA_TOPKB_CASE(4);
    else if (E <= 256) XMA_TOPKB_CASE(8);
    else if (E <= 512) XMA_TOPKB_CASE(16);
    else XMA_TOPKB_CASE(32);
#undef XMA_TOPKB_CASE
    return static_cast<int>(cudaGetLastError());
}

}  // namespace xma

namespace {
template <typename IdT>
int count_sort_impl(const IdT* ids, int64_t n, int E, uint32_t* counts, int* offsets_incl, int* pad_offsets,
                    int* tile_prefix, int* tile_expert, int64_t tile_cap, int* sorted_expert, int* sorted_scattered,
                    int* row_src, int64_t row_cap, int* row_dst, void* scratch, int64_t scratch_bytes,
                    int* device_status, cudaStream_t stream) {
    XMA_CUDA_TRY(cudaMemsetAsync(counts, 0, sizeof(uint32_t) * E, stream));
    const int64_t tiles = xma::ceil_div(n, xma::SORT_TILE);
    const xma::SortScratch sc = xma::sort_scratch_layout(static_cast<unsigned char*>(scratch), n, E);
    if (n > 0) {
        XMA_CUDA_TRY(cudaMemsetAsync(scratch, 0, sc.bytes, stream));
        int copies = static_cast<int>((40 * 1024) / (static_cast<int64_t>(E) * sizeof(unsigned)));
        copies = copies < 1 ? 1 : (copies > xma::SORT_WARPS ? xma::SORT_WARPS : copies);
        const int64_t cap = static_cast<int64_t>(xma::num_sms()) * 4;
        const int grid = static_cast<int>(tiles < cap ? tiles : cap);
        xma::tile_histogram_kernel<IdT><<<grid, xma::SORT_THREADS, static_cast<size_t>(copies + 1) * E * sizeof(unsigned),
                                         stream>>>(ids, n, E, copies, sc.tile_counts, counts, device_status);
        XMA_CUDA_TRY(cudaGetLastError());
    }
    xma::plan_kernel<<<1, 1024, 0, stream>>>(counts, E, offsets_incl, pad_offsets, tile_prefix, tile_expert,
                                            static_cast<int>(tile_cap), row_src, n == 0 ? 1 : 0, device_status);
    XMA_CUDA_TRY(cudaGetLastError());
    (void)row_cap;
    if (n == 0) return XMA_OK;
    const int64_t chunks = xma::ceil_div(tiles, static_cast<int64_t>(xma::SCAN_TILES));
    xma::tile_scan_kernel<<<static_cast<int>(chunks), xma::SCAN_THREADS, 0, stream>>>(
        sc, tiles, E, offsets_incl, counts, tile_prefix, tile_expert, static_cast<int>(tile_cap), row_src,
        device_status);
    XMA_CUDA_TRY(cudaGetLastError());
    const size_t smem = xma::sort_smem_bytes(E);
    int bits = 1;
    while ((1 << bits) < E) ++bits;  // bits of the largest bin index E - 1
    const int passes = (bits + xma::RADIX_BITS - 1) / xma::RADIX_BITS;
    (void)scratch_bytes;
    auto kernel = xma::sort_scatter_kernel<IdT>;
    XMA_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    kernel<<<static_cast<int>(tiles), xma::SORT_THREADS, smem, stream>>>(
        ids, n, E, passes, offsets_incl, pad_offsets, sorted_expert, sorted_scattered, row_src, row_dst, sc,
        device_status);
    return static_cast<int>(cudaGetLastError());
}
}  // namespace

// ================================================================================================
// C ABI
// ================================================================================================
extern "C" {

int xma_b200_continuous_count(const void* ids, int id_dtype, int64_t n, int bins, uint32_t* counts,
                              int* device_status, cudaStream_t stream) {
    if (!counts || (n > 0 && !ids)) return XMA_ERR_NULL_POINTER;
    if (n < 0 || bins <= 0) return XMA_ERR_BAD_SHAPE;
    if (id_dtype == XMA_I32) {
        if (reinterpret_cast<uintptr_t>(ids) & 3u) return XMA_ERR_MISALIGNED;
        return xma::launch_histogram(static_cast<const int*>(ids), n, bins, counts, device_status, stream);
    }
    if (id_dtype == XMA_I64) {
        if (reinterpret_cast<uintptr_t>(ids) & 7u) return XMA_ERR_MISALIGNED;
        return xma::launch_histogram(static_cast<const long long*>(ids), n, bins, counts, device_status, stream);
    }
    return XMA_ERR_BAD_DTYPE;
}

int64_t xma_b200_count_sort_scratch_bytes(int64_t n, int num_experts) {
    if (n < 0 || num_experts <= 0 || num_experts > xma::SORT_MAX_BINS) return XMA_ERR_BAD_SHAPE;
    return static_cast<int64_t>(xma::sort_scratch_bytes(n, num_experts));
}

int64_t xma_b200_tile_capacity(int64_t n, int num_experts) {
    if (n < 0 || num_experts <= 0) return XMA_ERR_BAD_SHAPE;
    return n / XMA_ROW_PAD + num_experts;
}


int xma_b200_count_sort(const void* ids, int id_dtype, int64_t n, int num_experts, uint32_t* counts,
                        int32_t* offsets_incl, int32_t* pad_offsets, int32_t* tile_prefix, int32_t* tile_expert,
                        int64_t tile_cap, int32_t* sorted_expert_idxs, int32_t* sorted_scattered_idxs,
                        int32_t* row_src, int64_t row_cap, int32_t* row_dst, void* scratch, int64_t scratch_bytes,
                        int* device_status, cudaStream_t stream) {
    if (!counts || !offsets_incl || !pad_offsets || !tile_prefix || !tile_expert || !scratch ||
        (n > 0 && (!ids || !sorted_expert_idxs || !sorted_scattered_idxs)))
        return XMA_ERR_NULL_POINTER;
    if (n < 0 || num_experts <= 0 || num_experts > xma::SORT_MAX_BINS) return XMA_ERR_BAD_SHAPE;
    if (n > 0x7fffffffLL - xma::SORT_TILE) return XMA_ERR_TOO_LARGE;
    if (tile_cap < n / XMA_ROW_PAD + num_experts) return XMA_ERR_BAD_SHAPE;
    if (row_src && row_cap < tile_cap * XMA_ROW_PAD) return XMA_ERR_BAD_SHAPE;
    if (scratch_bytes < static_cast<int64_t>(xma::sort_scratch_bytes(n, num_experts))) return XMA_ERR_SCRATCH_TOO_SMALL;
    if (reinterpret_cast<uintptr_t>(scratch) & 255u) return XMA_ERR_MISALIGNED;
    if (id_dtype == XMA_I32)
        return count_sort_impl(static_cast<const int*>(ids), n, num_experts, counts, offsets_incl, pad_offsets,
                               tile_prefix, tile_expert, tile_cap, sorted_expert_idxs, sorted_scattered_idxs,
                               row_src, row_cap, row_dst, scratch, scratch_bytes, device_status, stream);
    if (id_dtype == XMA_I64)
        return count_sort_impl(static_cast<const long long*>(ids), n, num_experts, counts, offsets_incl,
                               pad_offsets, tile_prefix, tile_expert, tile_cap, sorted_expert_idxs,
                               sorted_scattered_idxs, row_src, row_cap, row_dst, scratch, scratch_bytes,
                               device_status, stream);
    return XMA_ERR_BAD_DTYPE;
}

int xma_b200_route_topk_softmax(const void* logits, int dtype, int64_t logits_row_stride, int64_t tokens,
                                int num_experts, int top_k, void* weights, int32_t* selected_i32,
                                int64_t* selected_i64, cudaStream_t stream) {
    if (tokens > 0 && (!logits || !weights || (!selected_i32 && !selected_i64))) return XMA_ERR_NULL_POINTER;
    if (tokens < 0 || num_experts <= 0 || num_experts > 1024 || top_k <= 0 || top_k > 32 || top_k > num_experts ||
        logits_row_stride < num_experts)
        return XMA_ERR_BAD_SHAPE;
    long long* s64 = reinterpret_cast<long long*>(selected_i64);
    switch (dtype) {
        case XMA_F32:
            return xma::launch_topk<float>(logits, logits_row_stride, tokens, num_experts, top_k, weights,
                                           selected_i32, s64, stream);
        case XMA_F16:
            return xma::launch_topk<__half>(logits, logits_row_stride, tokens, num_experts, top_k, weights,
                                            selected_i32, s64, stream);
        case XMA_BF16:
            return xma::launch_topk<__nv_bfloat16>(logits, logits_row_stride, tokens, num_experts, top_k, weights,
                                                   selected_i32, s64, stream);
    }
    return XMA_ERR_BAD_DTYPE;
}

int xma_b200_route_topk_softmax_bwd(const void* logits, int dtype, int64_t logits_row_stride,
                                    const int32_t* selected_i32, const void* d_weights, int64_t tokens,
                                    int num_experts, int top_k, void* d_logits, cudaStream_t stream) {
    if (tokens > 0 && (!logits || !selected_i32 || !d_weights || !d_logits)) return XMA_ERR_NULL_POINTER;
    if (tokens < 0 || num_experts <= 0 || num_experts > 1024 || top_k <= 0 || top_k > 32 || top_k > num_experts ||
        logits_row_stride < num_experts)
        return XMA_ERR_BAD_SHAPE;
    switch (dtype) {
        case XMA_F32:
            return xma::launch_topk_bwd<float>(logits, logits_row_stride, selected_i32, d_weights, tokens,
                                               num_experts, top_k, d_logits, stream);
        case XMA_F16:
            return xma::launch_topk_bwd<__half>(logits, logits_row_stride, selected_i32, d_weights, tokens,
                                                num_experts, top_k, d_logits, stream);
        case XMA_BF16:
            return xma::launch_topk_bwd<__nv_bfloat16>(logits, logits_row_stride, selected_i32, d_weights, tokens,
                                                       num_experts, top_k, d_logits, stream);
    }
    return XMA_ERR_BAD_DTYPE;
}

}  // extern "C"

// ================================================================================================
// Counting sort without caller-provided scratch
// ================================================================================================
// Some hosts of this library must not allocate device memory while they run: a serving engine that
// has handed its whole memory budget to a pool at start-up, or a step that sits between other
// frameworks' allocators and may not disturb them. For those callers the sort's scratch (per-tile
// counts and the look-back words of the scan over them) lives in this fixed array instead of a caller
// buffer. Every GPU that loads the library holds it until the process exits.
#define XMA_STATIC_SORT_SCRATCH_BYTES (256 + 256 * 256 * 8) /* e.g. 480 tiles of 8192 ids x 256 experts */

static __device__ __align__(256) unsigned char g_static_sort_scratch[XMA_STATIC_SORT_SCRATCH_BYTES];

namespace {
constexpr int kMaxDevices = 64;
std::mutex g_static_scratch_mutex;
void* g_static_scratch_addr[kMaxDevices] = {nullptr};

cudaError_t preload_sort_kernels() {
    cudaFuncAttributes a;
    cudaError_t rc;
    if ((rc = cudaFuncGetAttributes(&a, xma::sort_scatter_kernel<int>)) != cudaSuccess) return rc;
    if ((rc = cudaFuncGetAttributes(&a, xma::sort_scatter_kernel<long long>)) != cudaSuccess) return rc;
    if ((rc = cudaFuncGetAttributes(&a, xma::tile_histogram_kernel<int>)) != cudaSuccess) return rc;
    if ((rc = cudaFuncGetAttributes(&a, xma::tile_histogram_kernel<long long>)) != cudaSuccess) return rc;
    if ((rc = cudaFuncGetAttributes(&a, xma::tile_scan_kernel)) != cudaSuccess) return rc;
    return cudaFuncGetAttributes(&a, xma::plan_kernel);
}
}  // namespace

extern "C" {

// Largest scratch the static variant can serve; the scratch a call needs is
// xma_b200_count_sort_scratch_bytes(n, num_experts).
int64_t xma_b200_count_sort_static_scratch_limit(void) { return XMA_STATIC_SORT_SCRATCH_BYTES; }

// Same outputs as xma_b200_count_sort, bit for bit, with the scratch taken from the library's own
// fixed device array. Nothing is allocated or freed, here or in anything this calls.
//  - The first call on each device looks up the array's device address (the name is only a host-side
//    handle, not an address a kernel could use) with that device current; make that first call
//    before any stream capture begins. With CUDA's lazy module loading that first use may also be the
//    moment the driver loads this library's code and the array onto the device (a driver-side
//    allocation of the module image): issue it at start-up, before a pool takes the memory budget.
//  - All calls on a device share the one array. It is cleared at the start of every call; two calls
//    whose kernels overlap on the GPU (different streams, no ordering) would corrupt each other.
//  - Problems whose scratch exceeds the limit are refused with XMA_ERR_TOO_LARGE.
int xma_b200_count_sort_static(const void* ids, int id_dtype, int64_t n, int num_experts, uint32_t* counts,
                               int32_t* offsets_incl, int32_t* pad_offsets, int32_t* tile_prefix,
                               int32_t* tile_expert, int64_t tile_cap, int32_t* sorted_expert_idxs,
                               int32_t* sorted_scattered_idxs, int32_t* row_src, int64_t row_cap,
                               int* device_status, cudaStream_t stream) {
    if (n < 0 || num_experts <= 0 || num_experts > xma::SORT_MAX_BINS) return XMA_ERR_BAD_SHAPE;
    const int64_t need = static_cast<int64_t>(xma::sort_scratch_bytes(n, num_experts));
    if (need > XMA_STATIC_SORT_SCRATCH_BYTES) return XMA_ERR_TOO_LARGE;
    int dev = -1;
    XMA_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) return XMA_ERR_UNSUPPORTED;
    void* scratch = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
        if (!g_static_scratch_addr[dev]) {
            void* p = nullptr;
            XMA_CUDA_TRY(cudaGetSymbolAddress(&p, g_static_sort_scratch));
            // every kernel a later call may launch is loaded now, so that lazy loading cannot allocate behind a
            // later call
            XMA_CUDA_TRY(preload_sort_kernels());
            g_static_scratch_addr[dev] = p;
        }
        scratch = g_static_scratch_addr[dev];
    }
    return xma_b200_count_sort(ids, id_dtype, n, num_experts, counts, offsets_incl, pad_offsets, tile_prefix,
                               tile_expert, tile_cap, sorted_expert_idxs, sorted_scattered_idxs, row_src, row_cap,
                               nullptr, scratch, XMA_STATIC_SORT_SCRATCH_BYTES, device_status, stream);
}

}  // extern "C"
