// Output-stationary MVMR on sm_100a: the fp32 sums of a block of 128 output rows stay in
// tensor memory (TMEM) across ALL taps and every output row is rounded and written exactly
// once -- no fp32 accumulator in global memory, no zero-fill, no rounding pass, no atomics,
// and a result that does not depend on the order in which CTAs run.
//
// The schedule needs the rulebook regrouped by output row.  That is done once per rulebook
// and direction by pcx_mvmr_plan_build into a caller-owned "plan":
//
//   rows     output rows are ordered by their tap signature (the set of taps that touch the
//            row) and, for a cubic kernel of at most 32 taps, first by the kernel planes that
//            set spans, so that the 128 rows of a block use few distinct taps and the
//            (block, tap) tiles below are well filled; perm[block * 128 + slot] = row
//   tiles    per (block, tap) a table of 128 source rows, one per slot: a feature row, "none",
//            or a row of the per-call scratch that holds the SUM of the feature rows of a
//            (row, tap) bucket with several triplets (the bucket pre-sum of the reference's fused
//            gather-sum schedule, sparse_engines/fused_point_conv.py:344-423); tile_offs is the
//            dense (nblocks * K + 1) table of triplet counts that tells which tiles exist
//   entries  per triplet (slot | position in its bucket << 8, feature row), ordered by
//            (block, tap, slot): the members of a bucket are consecutive
//   buckets  (first entry, length) of every bucket with more than one triplet
//   groups   G consecutive blocks share the weight tiles they stream; groups are handed out
//            most expensive first (a ticket counter inside the plan)
//
// Per call: a small kernel sums the rows of the multi-triplet buckets into the scratch (fp32 sum,
// one rounding), then the main kernel (TMEM columns = G accumulators of out_width fp32 each):
//
//   producer warps   together, one (block, tap, 64-channel slice) A tile after the other: every
//                    thread issues its 16-byte cp.async copies of the tile's source rows straight
//                    into the 128-byte-swizzled slot (rows without a source are zero-filled by the
//                    same instruction with a source size of 0); a tile is handed to the tensor
//                    core two tiles later, when its copies have landed anyway, with one mbarrier
//                    arrival per warp; the copies of several tiles are in flight at any time
//   weight warp      streams the 64-channel slices of W[tap] through a small ring with TMA
//                    (cp.async.bulk.tensor tile loads, 128-byte swizzle); one slice serves
//                    all blocks of the group that use the tap
//   MMA warp         one thread issues tcgen05.mma (M = 128 rows, N = out_width, K = 16 per
//                    instruction) with accumulate = 1 from the block's second tile on;
//                    tcgen05.commit releases the A slot, the weight slot and finally hands
//                    the accumulators to the epilogue
//   epilogue         the producer warps read TMEM (tcgen05.ld), round once and write each
//                    output row with 16-byte stores
//
// Every wait is bounded (one second) and abortable: a role that gives up raises a flag in the
// status word and in shared memory, the other roles leave their waits, and the CTA frees its
// TMEM and returns.
#include <cub/cub.cuh>
#include <cuda.h>

#include "sparse_kernels.cuh"
#include "tcgen05.cuh"

namespace pcx {
int device_status_address(unsigned int **d_status);

namespace {

using namespace tc;

constexpr int ROWS = 128;             // output rows per block (the M of the MMA)
constexpr int SLOT_BYTES = ROWS * 128;  // one A tile: 128 rows of a 64-channel slice
constexpr int MAX_NPW = 8;            // producer warps
constexpr int MAX_SLOTS = 12;         // A slots
constexpr int MAX_NW = 4;             // weight slots
constexpr int MAX_GROUP = 8;          // blocks per group
constexpr int MAX_TAPS = 512;         // taps the shared-memory tables are sized for
constexpr int SIGNAL_LAG = 2;          // a tile is handed to the tensor core once the copies of the two tiles after it are issued
constexpr int ROW_PREFETCH = 1;        // tiles whose source rows a producer thread holds ahead of the one it issues (deeper did not pay: the copies, not this table, bound the producer)
constexpr int ROW_PASSES = 8;         // rows a producer thread copies per tile, at most (128 rows / (4 warps * 4 row lanes))
constexpr unsigned STATUS_BIT = 4u;   // bit of the device status word this kernel raises
constexpr unsigned PLAN_MAGIC = 0x70637832u;

// control words at the head of a plan
enum { CTRL_TICKET = 0, CTRL_DONE = 1, CTRL_MAGIC = 2, CTRL_GROUP = 3, CTRL_NMULTI = 4, CTRL_WORDS = 64 };

struct PlanView {
    uint32_t *ctrl;        // CTRL_WORDS
    int32_t *perm;         // nblocks * ROWS, -1 = padding
    int32_t *tile_offs;    // nblocks * K + 1
    uint2 *entries;        // T
    int32_t *group_order;  // ngroups
    int32_t *tile_rows;    // nblocks * K * ROWS: source row of (tile, slot): >= 0 feature row, -1 none, <= -2 scratch row -2 - x
    uint2 *buckets;        // T / 2 + 1: (first entry, length) of the buckets with several triplets
    int64_t nblocks, ngroups;
};

size_t carve_plan(void *base, int64_t T, int64_t n_out, int K, int G, PlanView *out) {
    Carver c(base);
    PlanView v;
    v.nblocks = (n_out + ROWS - 1) / ROWS;
    v.ngroups = (v.nblocks + G - 1) / G;
    v.ctrl = c.take<uint32_t>(CTRL_WORDS);
    v.perm = c.take<int32_t>((size_t)v.nblocks * ROWS);
    v.tile_offs = c.take<int32_t>((size_t)v.nblocks * K + 1);
    v.entries = c.take<uint2>((size_t)std::max<int64_t>(T, 1));
    v.group_order = c.take<int32_t>((size_t)std::max<int64_t>(v.ngroups, 1));
    v.tile_rows = c.take<int32_t>((size_t)v.nblocks * K * ROWS);
    v.buckets = c.take<uint2>((size_t)(T / 2 + 1));
    if (out) *out = v;
    return c.off;
}

int bits_of(int64_t n) {
    int bits = 1;
    while (((int64_t)1 << bits) < n) ++bits;
    return bits;
}

struct BuildWs {
    uint32_t *sig, *sig_sorted;          // n_out
    int32_t *row, *row_sorted, *rank;    // n_out
    uint32_t *key, *key_sorted;          // T
    int32_t *val, *val_sorted;           // T
    int32_t *tile_cnt;                   // nblocks * K + 1
    uint32_t *cost, *cost_sorted;        // ngroups
    int32_t *gid;                        // ngroups
    void *cub_tmp;
    size_t cub_bytes;
};

size_t carve_build(void *base, int64_t T, int64_t n_out, int K, int G, BuildWs *out) {
    Carver c(base);
    BuildWs w;
    const int64_t nblocks = (n_out + ROWS - 1) / ROWS, ngroups = (nblocks + G - 1) / G;
    const size_t n = (size_t)std::max<int64_t>(n_out, 1), t = (size_t)std::max<int64_t>(T, 1);
    const size_t g = (size_t)std::max<int64_t>(ngroups, 1);
    w.sig = c.take<uint32_t>(n), w.sig_sorted = c.take<uint32_t>(n);
    w.row = c.take<int32_t>(n), w.row_sorted = c.take<int32_t>(n), w.rank = c.take<int32_t>(n);
    w.key = c.take<uint32_t>(t), w.key_sorted = c.take<uint32_t>(t);
    w.val = c.take<int32_t>(t), w.val_sorted = c.take<int32_t>(t);
    w.tile_cnt = c.take<int32_t>((size_t)nblocks * K + 1);
    w.cost = c.take<uint32_t>(g), w.cost_sorted = c.take<uint32_t>(g);
    w.gid = c.take<int32_t>(g);
    size_t b1 = 0, b2 = 0, b3 = 0, b4 = 0;
    cub::DeviceRadixSort::SortPairs(nullptr, b1, (const uint32_t *)nullptr, (uint32_t *)nullptr, (const int32_t *)nullptr,
                                    (int32_t *)nullptr, (int)n, 0, 32);
    cub::DeviceRadixSort::SortPairs(nullptr, b2, (const uint32_t *)nullptr, (uint32_t *)nullptr, (const int32_t *)nullptr,
                                    (int32_t *)nullptr, (int)t, 0, 32);
    cub::DeviceScan::ExclusiveSum(nullptr, b3, (const int32_t *)nullptr, (int32_t *)nullptr, (int)((size_t)nblocks * K + 1));
    cub::DeviceRadixSort::SortPairsDescending(nullptr, b4, (const uint32_t *)nullptr, (uint32_t *)nullptr,
                                              (const int32_t *)nullptr, (int32_t *)nullptr, (int)g, 0, 32);
    w.cub_bytes = std::max(std::max(b1, b2), std::max(b3, b4));
    w.cub_tmp = c.take<char>(w.cub_bytes);
    if (out) *out = w;
    return c.off;
}

__device__ __forceinline__ uint32_t pack2(float a, float b, int fmt) {
    if (fmt) {
        __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
        return *reinterpret_cast<uint32_t *>(&v);
    }
    __half2 v = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t *>(&v);
}

__device__ __forceinline__ int tap_of(const int64_t *__restrict__ seg, int K, int64_t t) {
    int lo = 0, hi = K;  // last k with seg[k] <= t
    while (hi - lo > 1) {
        int mid = (lo + hi) >> 1;
        if (seg[mid] <= t) lo = mid; else hi = mid;
    }
    return lo;
}

__global__ void plan_init_kernel(int64_t n_out, uint32_t *sig, int32_t *row, int32_t *tile_cnt, int64_t n_tiles,
                                 uint32_t *ctrl, int G) {
    const int64_t x = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (x < n_out) sig[x] = 0u, row[x] = (int32_t)x;
    if (x <= n_tiles) tile_cnt[x] = 0;
    if (x < CTRL_WORDS) ctrl[x] = x == CTRL_MAGIC ? PLAN_MAGIC : x == CTRL_GROUP ? (uint32_t)G : 0u;
}

// Tap signature of every output row.  With more than 32 taps the taps are folded onto 32
// bits (tap mod 32): rows that share a signature then share a superset of taps.
__global__ void plan_sig_kernel(const int32_t *__restrict__ scatter, const int64_t *__restrict__ seg, int64_t T, int K,
                                uint32_t *sig) {
    const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= T) return;
    atomicOr(&sig[scatter[t]], 1u << (tap_of(seg, K, t) & 31));
}

// Second sort key of the rows of a cubic kernel (K = ks^3 <= 32 taps, tap = (kx * ks + ky) * ks + kz):
// which kx / ky / kz planes of the kernel a row uses at all, kz most significant.  Points of a
// scene lie on surfaces; rows of one surface orientation share these planes even where their
// exact tap sets differ, and sorted by (planes, signature) the blocks of 128 rows need a quarter
// fewer (block, tap) tiles on thin rulebooks than sorted by signature alone.
__global__ void plan_planes_kernel(const uint32_t *__restrict__ sig_sorted, int64_t n_out, int K, int ks, uint32_t *planes) {
    const int64_t x = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (x >= n_out) return;
    const uint32_t m = sig_sorted[x];
    uint32_t px = 0, py = 0, pz = 0;
    for (int tap = 0; tap < K; ++tap)
        if ((m >> tap) & 1u) px |= 1u << (tap / (ks * ks)), py |= 1u << ((tap / ks) % ks), pz |= 1u << (tap % ks);
    planes[x] = px | (py << ks) | (pz << (2 * ks));
}

__global__ void plan_rank_kernel(const int32_t *__restrict__ row_sorted, int64_t n_out, int64_t n_pad, int32_t *rank,
                                 int32_t *perm) {
    const int64_t x = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (x >= n_pad) return;
    if (x < n_out) {
        const int32_t r = row_sorted[x];
        rank[r] = (int32_t)x;
        perm[x] = r;
    } else {
        perm[x] = -1;
    }
}

__global__ void plan_keys_kernel(const int32_t *__restrict__ scatter, const int32_t *__restrict__ gather,
                                 const int64_t *__restrict__ seg, const int32_t *__restrict__ rank, int64_t T, int K,
                                 uint32_t *key, int32_t *val, int32_t *tile_cnt) {
    const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= T) return;
    const int k = tap_of(seg, K, t);
    const uint32_t r = (uint32_t)rank[scatter[t]];
    const uint32_t tile = (r >> 7) * (uint32_t)K + (uint32_t)k;
    key[t] = (tile << 7) | (r & 127u);
    val[t] = gather[t];
    atomicAdd(&tile_cnt[tile], 1);
}

// entries[t] = (slot | position within the (row, tap) bucket << 8, feature row); the first entry
// of a bucket also fills the bucket's slot of its tile's row table: the feature row itself, or,
// when more triplets follow, the scratch row the bucket's sum will be written to
__global__ void plan_entries_kernel(const uint32_t *__restrict__ key_sorted, const int32_t *__restrict__ val_sorted,
                                    int64_t T, uint2 *entries, int32_t *tile_rows, uint2 *buckets, uint32_t *ctrl) {
    const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= T) return;
    const uint32_t k = key_sorted[t];
    uint32_t pos = 0;
    while (pos < 0xffffffu && t - (int64_t)pos - 1 >= 0 && key_sorted[t - pos - 1] == k) ++pos;
    entries[t] = make_uint2((k & 127u) | (pos << 8), (uint32_t)val_sorted[t]);
    if (pos != 0) return;
    uint32_t len = 1;
    while (t + len < T && key_sorted[t + len] == k) ++len;
    if (len == 1) {
        tile_rows[k] = val_sorted[t];   // key = tile * 128 + slot
    } else {
        const uint32_t b = atomicAdd(&ctrl[CTRL_NMULTI], 1u);
        buckets[b] = make_uint2((uint32_t)t, len);
        tile_rows[k] = -2 - (int32_t)b;
    }
}

// scratch[b] = sum of the feature rows of bucket b (fp32 sum in entry order, one rounding); one thread
// per 16-byte piece.  The row indices of up to four members are fetched together and their pieces
// together after that, so that a bucket costs two memory latencies instead of two per member.
// The element format and, for the usual row widths, the pieces per row are compile-time values: the
// first version of this kernel spent most of its instructions on a 64-bit division of the thread
// index and on per-element format branches (749 M warp instructions for 9 M buckets, issue-bound
// at 28 % of the DRAM bandwidth).
template <int FMT>
__device__ __forceinline__ void add_piece(float (&acc)[8], uint4 v) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        float2 f;
        if (FMT) f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&w[q]));
        else f = __half22float2(*reinterpret_cast<const __half2 *>(&w[q]));
        acc[2 * q] += f.x, acc[2 * q + 1] += f.y;
    }
}

constexpr int BUCKET_SUM_THREADS = 256;

// PPR: 16-byte pieces per row when that is a power of two (2 .. 32), else 0 (taken from inw).
// (Two pieces per thread were tried: fewer instructions per byte, but fewer resident warps, and slower.)
template <int FMT, int PPR>
__global__ void __launch_bounds__(BUCKET_SUM_THREADS) bucket_sum_kernel(const uint16_t *__restrict__ feat,
                                                                        const uint2 *__restrict__ entries,
                                                                        const uint2 *__restrict__ buckets,
                                                                        const uint32_t *__restrict__ ctrl, int inw,
                                                                        uint16_t *scratch) {
    const unsigned ppr = PPR ? (unsigned)PPR : (unsigned)inw >> 3;
    const unsigned per_block = BUCKET_SUM_THREADS / ppr;
    const unsigned local = threadIdx.x / ppr, piece = threadIdx.x - local * ppr;
    const unsigned b = blockIdx.x * per_block + local;
    if (local >= per_block || b >= ctrl[CTRL_NMULTI]) return;
    const uint2 bk = __ldg(buckets + b);
    const uint16_t *col = feat + piece * 8;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (uint32_t m0 = 0; m0 < bk.y; m0 += 4) {
        uint32_t rows[4];
#pragma unroll
        for (int m = 0; m < 4; ++m) rows[m] = m0 + m < bk.y ? __ldg(&entries[bk.x + m0 + m].y) : 0u;
        uint4 v[4];
#pragma unroll
        for (int m = 0; m < 4; ++m)
            v[m] = m0 + m < bk.y ? __ldg(reinterpret_cast<const uint4 *>(col + (size_t)rows[m] * (unsigned)inw)) : make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int m = 0; m < 4; ++m) add_piece<FMT>(acc, v[m]);   // an absent member adds zeros
    }
    uint4 o;
    o.x = pack2(acc[0], acc[1], FMT), o.y = pack2(acc[2], acc[3], FMT);
    o.z = pack2(acc[4], acc[5], FMT), o.w = pack2(acc[6], acc[7], FMT);
    *reinterpret_cast<uint4 *>(scratch + (size_t)b * (unsigned)inw + piece * 8) = o;
}

template <int FMT>
void launch_bucket_sum(int64_t multi, int inw, const uint16_t *feat, const uint2 *entries, const uint2 *buckets,
                       const uint32_t *ctrl, uint16_t *scratch, cudaStream_t stream) {
    const int ppr = inw >> 3;
    const unsigned grid = (unsigned)((multi + BUCKET_SUM_THREADS / ppr - 1) / (BUCKET_SUM_THREADS / ppr));
#define PCX_BS(P) bucket_sum_kernel<FMT, P><<<grid, BUCKET_SUM_THREADS, 0, stream>>>(feat, entries, buckets, ctrl, inw, scratch)
    switch (ppr) {
        case 2: PCX_BS(2); break;
        case 4: PCX_BS(4); break;
        case 8: PCX_BS(8); break;
        case 16: PCX_BS(16); break;
        case 32: PCX_BS(32); break;
        default: PCX_BS(0); break;
    }
#undef PCX_BS
}

// cost of a group = its non-empty tiles (each is one A tile to gather and multiply)
__global__ void plan_cost_kernel(const int32_t *__restrict__ tile_offs, int64_t nblocks, int K, int G, int64_t ngroups,
                                 uint32_t *cost, int32_t *gid) {
    const int64_t g = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (g >= ngroups) return;
    const int64_t t0 = g * G * K, t1 = min((g + 1) * (int64_t)G, nblocks) * K;
    uint32_t c = 0;
    for (int64_t x = t0; x < t1; ++x) c += tile_offs[x + 1] > tile_offs[x];
    cost[g] = c;
    gid[g] = (int32_t)g;
}

// ------------------------------------------------------------------ kernel ----

struct OsParams {
    const uint16_t *feat;
    uint16_t *out;
    const uint16_t *weight;
    const int32_t *perm, *tile_offs, *group_order, *tile_rows;
    const uint16_t *scratch;   // sums of the multi-triplet buckets
    const uint2 *entries;
    uint32_t *ctrl;
    unsigned int *status;
    int K, C, M, transpose, fmt;
    int inw, outw, nkb, G, ngroups, nblocks;
    int npw, nslots, nw, use_tma;
    int lag;   // 0: every thread's copies report to the slot's barrier themselves; SIGNAL_LAG: one arrival per warp, SIGNAL_LAG tiles later
    uint32_t w_slot_bytes, w_box_rows, w_tx_bytes;
    uint32_t ncols, col_stride;
    uint64_t wait_limit_ns;
};

__device__ __forceinline__ uint4 ldg_nc_v4(const void *p) {
    uint4 v;
    asm volatile("ld.global.nc.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ uint2 ldg_nc_v2(const void *p) {
    uint2 v;
    asm volatile("ld.global.nc.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
    return v;
}
__device__ __forceinline__ void sts_v4(uint32_t addr, uint4 v) {
    asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ uint4 lds_v4(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr) : "memory");
    return v;
}

// Optional cycle accounting per role (compile with -DPCX_OS_STATS): sums of clock64() spans are
// added to the plan's spare control words 8.. and read back by the caller.
#ifdef PCX_OS_STATS
#define STAT_T0(name) const long long name = clock64()
#define STAT_ADD(word, t0) do { if (lane == 0) atomicAdd(&p.ctrl[word], (uint32_t)((clock64() - (t0)) >> 4)); } while (0)
#else
#define STAT_T0(name)
#define STAT_ADD(word, t0)
#endif

// Task lists of a group, built in shared memory by the whole CTA before the roles start:
//   A task   one (block, tap, 64-channel slice) tile: its entries [lo, hi) and
//            meta = block | slice << 4 | first-of-slice << 8 | last-of-slice << 9 | tap << 16
//   W task   one (tap, slice) weight tile: tap | slice << 16
// Order (every role walks the same lists): taps ascending; per tap the slices of the
// contraction; per slice the blocks of the group that use the tap.
__device__ __forceinline__ int pieces_of(int inw, int q) { return min(8, (inw - q * 64) >> 3); }

__global__ void __launch_bounds__(512, 1)
mvmr_os_kernel(const __grid_constant__ CUtensorMap tmap, const OsParams p) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t s_a_full[MAX_SLOTS], s_a_empty[MAX_SLOTS], s_w_full[MAX_NW], s_w_empty[MAX_NW], s_d_full;
    __shared__ uint32_t s_tmem;
    __shared__ int s_group, s_ntiles, s_ntaps, s_abort;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t a_base = base, w_base = base + (uint32_t)p.nslots * SLOT_BYTES;
    uint8_t *tab_raw = smem_raw + (w_base + (uint32_t)p.nw * p.w_slot_bytes - smem_u32(smem_raw));
    // tables of the current group (16-byte aligned): A tasks, tile offsets, tile list, run ordinals, W tasks
    int4 *s_task = reinterpret_cast<int4 *>(tab_raw);                       // G*K*nkb
    int32_t *s_tab = reinterpret_cast<int32_t *>(s_task + p.G * p.K * p.nkb);  // G*K + 1
    int32_t *s_list = s_tab + (p.G * p.K + 1);                                // G*K: tap << 8 | block, tap-major
    int32_t *s_run = s_list + p.G * p.K;                                      // G*K: ordinal of the tile's tap among the group's taps
    int32_t *s_wtask = s_run + p.G * p.K;                                     // K*nkb
    volatile int *abort_flag = &s_abort;

    if (tid == 0) {
        for (int s = 0; s < p.nslots; ++s) mbar_init(smem_u32(&s_a_full[s]), (uint32_t)p.npw * (p.lag ? 1u : 32u)), mbar_init(smem_u32(&s_a_empty[s]), 1);
        for (int s = 0; s < p.nw; ++s) mbar_init(smem_u32(&s_w_full[s]), p.use_tma ? 1 : 32), mbar_init(smem_u32(&s_w_empty[s]), 1);
        mbar_init(smem_u32(&s_d_full), 1);
        fence_mbar_init();
        s_abort = 0;
        if (p.use_tma) tma_prefetch_desc(&tmap);
    }
    if (warp == 0) tmem_alloc(smem_u32(&s_tmem), p.ncols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = s_tmem;
    const uint32_t idesc = instr_desc(p.fmt, ROWS, p.outw, 0, p.transpose ? 0 : 1);

    // A tiles, weight tiles and accumulator hand-overs of the groups this CTA has finished (all
    // roles count alike): tile n uses A slot n mod nslots for the (n / nslots)-th time, and so on
    uint32_t a_n = 0, w_n = 0, d_n = 0;

    for (;;) {
        STAT_T0(t_group);
        if (tid == 0) {
            const uint32_t ticket = atomicAdd(&p.ctrl[CTRL_TICKET], 1u);
            s_group = ticket < (uint32_t)p.ngroups ? p.group_order[ticket] : -1;
        }
        __syncthreads();
        const int g = s_group;
        if (g < 0 || s_abort) break;
        const int b0 = g * p.G, nb = min(p.G, p.nblocks - b0);
        for (int x = tid; x <= nb * p.K; x += blockDim.x) s_tab[x] = p.tile_offs[(int64_t)b0 * p.K + x];
        __syncthreads();
        if (warp == 0) {  // the non-empty (tap, block) pairs, tap-major, and the ordinal of each pair's tap
            int count = 0;
            for (int x0 = 0; x0 < nb * p.K; x0 += 32) {
                const int x = x0 + lane;
                int tap = 0, blk = 0;
                bool has = false;
                if (x < nb * p.K) {
                    tap = x / nb, blk = x - tap * nb;
                    has = s_tab[blk * p.K + tap + 1] > s_tab[blk * p.K + tap];
                }
                const unsigned m = __ballot_sync(0xffffffffu, has);
                if (has) s_list[count + __popc(m & ((1u << lane) - 1u))] = (tap << 8) | blk;
                count += __popc(m);
            }
            __syncwarp();
            int taps = 0;
            for (int x0 = 0; x0 < count; x0 += 32) {
                const int x = x0 + lane;
                const bool head = x < count && (x == 0 || (s_list[x] >> 8) != (s_list[x - 1] >> 8));
                const unsigned m = __ballot_sync(0xffffffffu, head);
                if (x < count) s_run[x] = taps + __popc(m & (0xffffffffu >> (31 - lane))) - 1;
                taps += __popc(m);
            }
            if (lane == 0) s_ntiles = count, s_ntaps = taps;
        }
        __syncthreads();
        const int ntiles = s_ntiles, a_total = ntiles * p.nkb, w_total = s_ntaps * p.nkb;
        for (int x = tid; x < ntiles; x += blockDim.x) {  // expand the tile list into the task lists
            const int tap = s_list[x] >> 8, blk = s_list[x] & 255;
            int r0 = x, r1 = x + 1;
            while (r0 > 0 && (s_list[r0 - 1] >> 8) == tap) --r0;
            while (r1 < ntiles && (s_list[r1] >> 8) == tap) ++r1;
            const int lo = s_tab[blk * p.K + tap], hi = s_tab[blk * p.K + tap + 1];
            for (int q = 0; q < p.nkb; ++q) {
                const int meta = blk | (q << 4) | ((x == r0) << 8) | ((x + 1 == r1) << 9) | (tap << 16);
                s_task[r0 * p.nkb + q * (r1 - r0) + (x - r0)] = make_int4(lo, hi, meta, 0);
                if (x == r0) s_wtask[s_run[x] * p.nkb + q] = tap | (q << 16);
            }
        }
        __syncthreads();

        if (warp == 0) STAT_ADD(8, t_group);
        STAT_T0(t_role);
        if (warp < p.npw) {
            // ---------------------------------------------------------- producer ----
            // All producer threads fill every tile together: 8 threads per row (one 16-byte piece
            // each), npw * 4 rows per pass.  The source rows of the next tile are fetched while
            // the current one is issued.
            const int piece = tid & 7, row_lane = tid >> 3, row_lanes = p.npw * 4, passes = ROWS / row_lanes;
            // row_lanes is a multiple of 8, so the rows of a thread share their low three bits and
            // with them the swizzled position of the thread's piece inside a row
            const uint32_t lane_offset = (uint32_t)row_lane * 128 + (uint32_t)((piece ^ (row_lane & 7)) << 4);
            const uint32_t pass_stride = (uint32_t)row_lanes * 128;
            uint32_t slot = a_n % (uint32_t)p.nslots, use = a_n / (uint32_t)p.nslots;
            uint32_t signal_slot = slot;   // slot of the oldest tile not handed over yet
            bool ok_role = true;
            // source rows of the next ROW_PREFETCH tiles: buffer u holds tile t with t mod ROW_PREFETCH == u
            // (static indexing: the loop below is unrolled by ROW_PREFETCH, so no register is moved
            // while its load is in flight)
            int rows_q[ROW_PREFETCH][ROW_PASSES];
            auto fetch_rows = [&](int task, int (&dst)[ROW_PASSES]) {
#pragma unroll
                for (int k = 0; k < ROW_PASSES; ++k) dst[k] = -1;
                if (task >= a_total) return;
                const int meta = s_task[task].z;
                const int32_t *table = p.tile_rows + ((int64_t)(b0 + (meta & 15)) * p.K + (meta >> 16)) * ROWS + row_lane;
#pragma unroll
                for (int k = 0; k < ROW_PASSES; ++k)
                    if (k < passes) dst[k] = __ldg(table + k * row_lanes);
            };
#pragma unroll
            for (int u = 0; u < ROW_PREFETCH; ++u) fetch_rows(u, rows_q[u]);
            for (int t0 = 0; t0 < a_total && ok_role; t0 += ROW_PREFETCH) {
#pragma unroll
              for (int u = 0; u < ROW_PREFETCH; ++u) {
                const int t = t0 + u;
                if (t >= a_total || !ok_role) break;
                int rows_cur[ROW_PASSES];
#pragma unroll
                for (int k = 0; k < ROW_PASSES; ++k) rows_cur[k] = rows_q[u][k];
                fetch_rows(t + ROW_PREFETCH, rows_q[u]);
                const int q = (s_task[t].z >> 4) & 15;
                const bool piece_ok = piece < pieces_of(p.inw, q);
                const uint16_t *feat_col = p.feat + q * 64 + piece * 8, *sum_col = p.scratch + q * 64 + piece * 8;
                const uint32_t dst0 = a_base + slot * SLOT_BYTES + lane_offset;
                // the tensor core has finished reading this slot's previous tile
                STAT_T0(t_w);
                ok_role = mbar_wait_abortable(smem_u32(&s_a_empty[slot]), (use & 1u) ^ 1u, STATUS_BIT, p.status, abort_flag,
                                              p.wait_limit_ns);
                STAT_ADD(9, t_w);
                if (!ok_role) break;
                if (piece_ok) {
#pragma unroll
                    for (int k = 0; k < ROW_PASSES; ++k) {
                        if (k < passes) {
                            const int src_row = rows_cur[k];
                            // a feature row, a row of bucket sums, or nothing (16 bytes of zeros: source size 0)
                            const uint16_t *src = src_row >= 0 ? feat_col + (int64_t)src_row * p.inw
                                                               : sum_col + (int64_t)(src_row == -1 ? 0 : -2 - src_row) * p.inw;
                            cp_async16_zfill(dst0 + (uint32_t)k * pass_stride, src_row == -1 ? (const void *)feat_col : (const void *)src,
                                             src_row == -1 ? 0u : 16u);
                        }
                    }
                }
                if (p.lag == 0) {
                    cp_async_mbar_arrive(smem_u32(&s_a_full[slot]));   // fires once this thread's copies have landed
                    if (++slot == (uint32_t)p.nslots) slot = 0, ++use;
                    continue;
                }
                cp_async_commit();
                // Hand over the tile issued SIGNAL_LAG tiles ago: its copies (a cp.async group of this
                // thread) have landed once at most SIGNAL_LAG newer groups are pending.  One arrival
                // per warp: an mbarrier takes arrivals one at a time, and one per thread and tile
                // would cost more than the copies.
                if (t >= SIGNAL_LAG) {
                    cp_async_wait<SIGNAL_LAG>();
                    fence_async_smem();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(smem_u32(&s_a_full[signal_slot]));
                    if (++signal_slot == (uint32_t)p.nslots) signal_slot = 0;
                }
                if (++slot == (uint32_t)p.nslots) slot = 0, ++use;
              }
            }
            // the last tiles of the group
            cp_async_wait<0>();
            fence_async_smem();
            __syncwarp();
            for (int t = max(a_total - SIGNAL_LAG, 0); t < a_total && ok_role && p.lag; ++t) {
                if (lane == 0) mbar_arrive(smem_u32(&s_a_full[signal_slot]));
                if (++signal_slot == (uint32_t)p.nslots) signal_slot = 0;
            }
            ok_role = __all_sync(0xffffffffu, ok_role);
            STAT_ADD(10, t_role);
            STAT_T0(t_epi);
            // ---------------------------------------------------------- epilogue ----
            if (ok_role && a_total > 0) {
                ok_role = mbar_wait_abortable(smem_u32(&s_d_full), d_n & 1u, STATUS_BIT, p.status, abort_flag, p.wait_limit_ns);
                ok_role = __all_sync(0xffffffffu, ok_role);
            }
            STAT_ADD(11, t_epi);
            tc_fence_after();
            const int teams = p.npw >> 2;
            if (ok_role && warp < teams * 4) {
                const int quarter = warp & 3, team = warp >> 2;
                const int chunks = p.outw >> 4;  // units of 16 columns
                for (int u = team; u < nb * chunks; u += teams) {
                    const int blk = u / chunks, cc = u - blk * chunks;
                    const int32_t row = p.perm[(int64_t)(b0 + blk) * ROWS + quarter * 32 + lane];
                    const bool blk_has = s_tab[(blk + 1) * p.K] > s_tab[blk * p.K];
                    float acc[16];
                    if (blk_has) {
                        tmem_ld16(tmem + ((uint32_t)(quarter * 32) << 16) + (uint32_t)blk * p.col_stride + (uint32_t)cc * 16, acc);
                    } else {
#pragma unroll
                        for (int c = 0; c < 16; ++c) acc[c] = 0.f;
                    }
                    if (row >= 0) {
                        uint4 *dst = reinterpret_cast<uint4 *>(p.out + (int64_t)row * p.outw + cc * 16);
                        uint4 o;
                        o.x = pack2(acc[0], acc[1], p.fmt), o.y = pack2(acc[2], acc[3], p.fmt);
                        o.z = pack2(acc[4], acc[5], p.fmt), o.w = pack2(acc[6], acc[7], p.fmt);
                        dst[0] = o;
                        o.x = pack2(acc[8], acc[9], p.fmt), o.y = pack2(acc[10], acc[11], p.fmt);
                        o.z = pack2(acc[12], acc[13], p.fmt), o.w = pack2(acc[14], acc[15], p.fmt);
                        dst[1] = o;
                    }
                }
            }
            tc_fence_before();
            STAT_ADD(12, t_epi);
        } else if (warp == p.npw) {
            // --------------------------------------------------------------- MMA ----
            if (lane == 0) {
                uint32_t slot = a_n % (uint32_t)p.nslots, use = a_n / (uint32_t)p.nslots;
                uint32_t wslot = w_n % (uint32_t)p.nw, wuse = w_n / (uint32_t)p.nw;
                uint32_t started = 0;
                bool ok_role = true;
                // descriptors of slot 0 / contraction step 0; the address field counts 16-byte units, so
                // another slot or step is an addition to the low word
                const uint64_t a_desc0 = smem_desc(a_base, 16, 1024);
                const uint64_t b_desc0 = p.transpose ? smem_desc(w_base, 16, 1024) : smem_desc(w_base, p.w_box_rows * 128, 1024);
                const uint32_t b_step = p.transpose ? 2u : 128u;  // 32 bytes along a K-major row / 16 contraction rows of 128 bytes
                const uint32_t w_slot16 = p.w_slot_bytes >> 4;
                for (int t = 0; t < a_total; ++t) {
                    const int meta = s_task[t].z;
                    const int blk = meta & 15, q = (meta >> 4) & 15;
                    if (meta & 256) {  // first tile of a weight slice: the slice has landed
                        STAT_T0(t_w);
                        ok_role = mbar_wait_abortable(smem_u32(&s_w_full[wslot]), wuse & 1u, STATUS_BIT, p.status, abort_flag,
                                                      p.wait_limit_ns);
                        if (!ok_role) break;
                        if (!p.use_tma) fence_async_smem();
                        STAT_ADD(13, t_w);
                    }
                    STAT_T0(t_a);
                    ok_role = mbar_wait_abortable(smem_u32(&s_a_full[slot]), use & 1u, STATUS_BIT, p.status, abort_flag,
                                                  p.wait_limit_ns);
                    if (!ok_role) break;
                    STAT_ADD(14, t_a);
                    fence_async_smem();   // the tile was written through the generic proxy, the tensor core reads through the async proxy
                    tc_fence_after();
                    const uint64_t ad = a_desc0 + (uint64_t)(slot * (SLOT_BYTES >> 4));
                    const uint64_t bd = b_desc0 + (uint64_t)(wslot * w_slot16);
                    const int ksteps = min(64, p.inw - q * 64) >> 4;
                    const uint32_t d_addr = tmem + (uint32_t)blk * p.col_stride;
                    const uint32_t first = (q > 0 || ((started >> blk) & 1u)) ? 1u : 0u;
                    STAT_T0(t_m);
                    tc_mma(d_addr, ad, bd, idesc, first);
                    for (int s = 1; s < ksteps; ++s) tc_mma(d_addr, ad + (uint64_t)(2 * s), bd + (uint64_t)(b_step * s), idesc, 1u);
                    STAT_ADD(18, t_m);
                    started |= 1u << blk;
                    STAT_T0(t_c);
                    tc_commit(smem_u32(&s_a_empty[slot]));
                    if (++slot == (uint32_t)p.nslots) slot = 0, ++use;
                    if (meta & 512) {  // last tile of the weight slice: its slot is free once these MMAs are done
                        tc_commit(smem_u32(&s_w_empty[wslot]));
                        if (++wslot == (uint32_t)p.nw) wslot = 0, ++wuse;
                    }
                    STAT_ADD(19, t_c);
                }
                if (ok_role && a_total > 0) tc_commit(smem_u32(&s_d_full));
                STAT_ADD(15, t_role);
            }
            __syncwarp();
        } else {
            // ------------------------------------------------------ weight loader ----
            uint32_t wslot = w_n % (uint32_t)p.nw, wuse = w_n / (uint32_t)p.nw;
            bool ok_role = true;
            for (int wt = 0; wt < w_total && ok_role; ++wt) {
                const int tap = s_wtask[wt] & 0xffff, q = s_wtask[wt] >> 16;
                const uint32_t w_slot = w_base + wslot * p.w_slot_bytes, full = smem_u32(&s_w_full[wslot]);
                STAT_T0(t_w);
                ok_role = mbar_wait_abortable(smem_u32(&s_w_empty[wslot]), (wuse & 1u) ^ 1u, STATUS_BIT, p.status, abort_flag,
                                              p.wait_limit_ns);
                ok_role = __all_sync(0xffffffffu, ok_role);
                STAT_ADD(16, t_w);
                if (!ok_role) break;
                if (p.use_tma) {
                    if (lane == 0) {
                        mbar_arrive_expect_tx(full, p.w_tx_bytes);
                        if (p.transpose) {
                            // contraction over m: the slice is the m-block q of all C rows of W[tap]
                            tma_load_2d(w_slot, &tmap, q * 64, tap * p.C, full);
                        } else {
                            // contraction over c: rows [64q, 64q + box) of W[tap], one box per 64 output channels
                            for (int mb = 0; mb * 64 < p.M; ++mb)
                                tma_load_2d(w_slot + (uint32_t)mb * p.w_box_rows * 128, &tmap, mb * 64, tap * p.C + q * 64, full);
                        }
                    }
                } else {
                    const uint16_t *w = p.weight + (int64_t)tap * p.C * p.M;
                    if (p.transpose) {
                        // rows c = 0..C-1, the 64 m-channels of block q (fewer in a last partial block)
                        const int cpr = min(8, (p.M - q * 64) >> 3);
                        for (int e = lane; e < p.C * cpr; e += 32) {
                            const int c = e / cpr, ch = e - c * cpr;
                            cp_async16(w_slot + (uint32_t)c * 128 + (uint32_t)((ch ^ (c & 7)) << 4),
                                       w + (int64_t)c * p.M + q * 64 + ch * 8);
                        }
                    } else {
                        // rows c = 64q .. 64q + rows - 1, all M channels in 64-channel blocks
                        const int rows = min(64, p.C - q * 64), cpr = p.M >> 3;
                        for (int e = lane; e < rows * cpr; e += 32) {
                            const int c = e / cpr, ch = e - c * cpr;
                            cp_async16(w_slot + (uint32_t)(ch >> 3) * p.w_box_rows * 128 + (uint32_t)c * 128 +
                                           (uint32_t)(((ch & 7) ^ (c & 7)) << 4),
                                       w + (int64_t)(q * 64 + c) * p.M + ch * 8);
                        }
                    }
                    cp_async_mbar_arrive(full);
                }
                if (++wslot == (uint32_t)p.nw) wslot = 0, ++wuse;
            }
        }
        if (warp == 0) STAT_ADD(17, t_group);
        // counters advance identically in every role
        a_n += (uint32_t)a_total;
        w_n += (uint32_t)w_total;
        d_n += a_total > 0 ? 1u : 0u;
        __syncthreads();
        if (s_abort) break;
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, p.ncols);
    // the last CTA to finish re-arms the ticket counter for the next launch
    if (tid == 0) {
        __threadfence();
        const uint32_t done = atomicAdd(&p.ctrl[CTRL_DONE], 1u);
        if (done == gridDim.x - 1) {
            p.ctrl[CTRL_TICKET] = 0u;
            p.ctrl[CTRL_DONE] = 0u;
            __threadfence();
        }
    }
}

// A single thread waits on an mbarrier that nothing arrives at: the bounded wait runs out,
// raises `flag` in the status word and the kernel returns.
__global__ void wait_runs_out_kernel(unsigned int *status, unsigned flag, uint64_t limit_ns) {
    __shared__ uint64_t s_bar;
    __shared__ int s_abort;
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&s_bar), 1);
        fence_mbar_init();
        s_abort = 0;
        mbar_wait_abortable(smem_u32(&s_bar), 0u, flag, status, &s_abort, limit_ns);
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// cuTensorMapEncodeTiled through the runtime's driver entry point table (the library does not
// link against libcuda); null when the driver does not offer it.
EncodeTiledFn encode_tiled() {
    static EncodeTiledFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void *ptr = nullptr;
        cudaDriverEntryPointQueryResult res;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &res) == cudaSuccess &&
            res == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)ptr;
        else
            (void)cudaGetLastError();
    }
    return fn;
}

unsigned int *status_word() {
    static unsigned int *ptr[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return nullptr;
    if (!ptr[dev & 63] && device_status_address(&ptr[dev & 63]) != PCX_OK) return nullptr;
    return ptr[dev & 63];
}

uint64_t wait_limit() {
    static uint64_t v = 0;
    if (!v) {
        const char *e = getenv("PCX_WAIT_LIMIT_NS");
        v = e ? strtoull(e, nullptr, 10) : 0;
        if (!v) v = WAIT_LIMIT_NS;
    }
    return v;
}

bool plan_sizes_ok(int64_t T, int64_t n_out, int K, int G) {
    if (T < 0 || T > INT32_MAX || n_out <= 0 || n_out > INT32_MAX || K <= 0 || K > MAX_TAPS) return false;
    if (G < 1 || G > MAX_GROUP) return false;
    const int64_t nblocks = (n_out + ROWS - 1) / ROWS;
    return nblocks * K * ROWS <= ((int64_t)1 << 32) && nblocks * K < INT32_MAX;
}

}  // namespace
}  // namespace pcx

using namespace pcx;

extern "C" {

int pcx_mvmr_plan_group_blocks(int out_width) {
    if (out_width <= 0 || out_width > 256) return 0;
    const int stride = (out_width + 31) / 32 * 32;
    // Two blocks per group, measured best at every width: up to 128 channels two accumulators fit
    // half of the tensor memory (two CTAs per SM), at 256 channels they fill it (one CTA per SM);
    // larger groups share each weight tile among more blocks but balance worse.
    int g = 2;
    if (const char *e = getenv("PCX_OS_GROUP")) {
        const int want = atoi(e);
        if (want >= 1 && want <= MAX_GROUP && want * stride <= 512) g = want;
    }
    return g;
}

size_t pcx_mvmr_plan_bytes(int64_t T, int64_t n_out, int K, int group_blocks) {
    if (!plan_sizes_ok(T, n_out, K, group_blocks)) return 0;
    return carve_plan(nullptr, T, n_out, K, group_blocks, nullptr);
}

size_t pcx_mvmr_plan_workspace_bytes(int64_t T, int64_t n_out, int K, int group_blocks) {
    if (!plan_sizes_ok(T, n_out, K, group_blocks)) return 0;
    return carve_build(nullptr, T, n_out, K, group_blocks, nullptr);
}

int pcx_mvmr_plan_build(const int32_t *d_scatter, const int32_t *d_gather, const int64_t *d_seg_offs, int64_t T, int K,
                        int64_t n_out, int group_blocks, void *d_plan, size_t plan_bytes, void *d_ws, size_t ws_bytes,
                        void *stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    const int G = group_blocks;
    if (!plan_sizes_ok(T, n_out, K, G))
        PCX_FAIL(PCX_E_UNSUPPORTED, "pcx_mvmr_plan_build: sizes out of range (T=%lld n_out=%lld K=%d group=%d)", (long long)T,
                 (long long)n_out, K, G);
    if (!d_plan || !d_ws || (T > 0 && (!d_scatter || !d_gather || !d_seg_offs)))
        PCX_FAIL(PCX_E_ARG, "pcx_mvmr_plan_build: null pointer");
    if ((uintptr_t)d_plan % 256 || (uintptr_t)d_ws % 256)
        PCX_FAIL(PCX_E_ALIGN, "pcx_mvmr_plan_build: plan and workspace must be 256-byte aligned");
    PlanView pv;
    BuildWs w;
    const size_t need_plan = carve_plan(d_plan, T, n_out, K, G, &pv), need_ws = carve_build(d_ws, T, n_out, K, G, &w);
    if (plan_bytes < need_plan) PCX_FAIL(PCX_E_CAPACITY, "pcx_mvmr_plan_build: plan buffer %zu < %zu bytes", plan_bytes, need_plan);
    if (ws_bytes < need_ws) PCX_FAIL(PCX_E_CAPACITY, "pcx_mvmr_plan_build: workspace %zu < %zu bytes", ws_bytes, need_ws);
    const int TPB = 256;
    const int64_t n_tiles = pv.nblocks * K, n_pad = pv.nblocks * ROWS;
    auto blocks = [&](int64_t n) { return (unsigned)((n + TPB - 1) / TPB); };
    const int64_t init_n = std::max<int64_t>(std::max<int64_t>(n_out, n_tiles + 1), CTRL_WORDS);
    PCX_CUDA(cudaMemsetAsync(pv.tile_rows, 0xff, (size_t)n_tiles * ROWS * sizeof(int32_t), stream));
    plan_init_kernel<<<blocks(init_n), TPB, 0, stream>>>(n_out, w.sig, w.row, w.tile_cnt, n_tiles, pv.ctrl, G);
    PCX_LAUNCH_CHECK();
    size_t bytes = w.cub_bytes;
    if (T > 0) {
        plan_sig_kernel<<<blocks(T), TPB, 0, stream>>>(d_scatter, d_seg_offs, T, K, w.sig);
        PCX_LAUNCH_CHECK();
    }
    // rows by signature (stable: rows of equal signature keep their order) ...
    PCX_CUDA(cub::DeviceRadixSort::SortPairs(w.cub_tmp, bytes, w.sig, w.sig_sorted, w.row, w.row_sorted, (int)n_out, 0,
                                             std::min(K, 32), stream));
    const int32_t *rows_in_order = w.row_sorted;
    int ks = 1;
    while (ks * ks * ks < K) ++ks;
    if (ks * ks * ks == K && K <= 32 && K > 1) {
        // ... and then, stable again, by the kernel planes they use: the order is (planes, signature)
        plan_planes_kernel<<<blocks(n_out), TPB, 0, stream>>>(w.sig_sorted, n_out, K, ks, w.sig);
        PCX_LAUNCH_CHECK();
        bytes = w.cub_bytes;
        PCX_CUDA(cub::DeviceRadixSort::SortPairs(w.cub_tmp, bytes, w.sig, w.sig_sorted, w.row_sorted, w.row, (int)n_out, 0,
                                                 3 * ks, stream));
        rows_in_order = w.row;
    }
    plan_rank_kernel<<<blocks(n_pad), TPB, 0, stream>>>(rows_in_order, n_out, n_pad, w.rank, pv.perm);
    PCX_LAUNCH_CHECK();
    if (T > 0) {
        plan_keys_kernel<<<blocks(T), TPB, 0, stream>>>(d_scatter, d_gather, d_seg_offs, w.rank, T, K, w.key, w.val, w.tile_cnt);
        PCX_LAUNCH_CHECK();
        bytes = w.cub_bytes;
        PCX_CUDA(cub::DeviceRadixSort::SortPairs(w.cub_tmp, bytes, w.key, w.key_sorted, w.val, w.val_sorted, (int)T, 0,
                                                 std::min(32, bits_of(n_tiles * ROWS)), stream));
    }
    bytes = w.cub_bytes;
    PCX_CUDA(cub::DeviceScan::ExclusiveSum(w.cub_tmp, bytes, w.tile_cnt, pv.tile_offs, (int)(n_tiles + 1), stream));
    if (T > 0) {
        plan_entries_kernel<<<blocks(T), TPB, 0, stream>>>(w.key_sorted, w.val_sorted, T, pv.entries, pv.tile_rows, pv.buckets,
                                                           pv.ctrl);
        PCX_LAUNCH_CHECK();
    }
    plan_cost_kernel<<<blocks(pv.ngroups), TPB, 0, stream>>>(pv.tile_offs, pv.nblocks, K, G, pv.ngroups, w.cost, w.gid);
    PCX_LAUNCH_CHECK();
    bytes = w.cub_bytes;
    PCX_CUDA(cub::DeviceRadixSort::SortPairsDescending(w.cub_tmp, bytes, w.cost, w.cost_sorted, w.gid, pv.group_order,
                                                       (int)pv.ngroups, 0, bits_of((int64_t)G * K + 2), stream));
    return PCX_OK;
}

size_t pcx_mvmr_planned_workspace_bytes(int64_t multi_buckets, int in_width) {
    if (multi_buckets < 0 || in_width <= 0) return 0;
    return align_up((size_t)std::max<int64_t>(multi_buckets, 1) * in_width * 2, 256);
}

int pcx_mvmr_plan_multi_buckets(const void *d_plan, int64_t *h_count, void *stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    if (!d_plan || !h_count) PCX_FAIL(PCX_E_ARG, "pcx_mvmr_plan_multi_buckets: null pointer");
    uint32_t n = 0;
    PCX_CUDA(cudaMemcpyAsync(&n, (const uint32_t *)d_plan + CTRL_NMULTI, sizeof(n), cudaMemcpyDeviceToHost, stream));
    PCX_CUDA(cudaStreamSynchronize(stream));
    *h_count = n;
    return PCX_OK;
}

int pcx_mvmr_planned(const void *d_weight, const void *d_feat, void *d_plan, size_t plan_bytes, void *d_out, int64_t T,
                     int64_t n_feat, int64_t n_out, int K, int C, int M, int transpose, int dtype, int group_blocks,
                     int64_t multi_buckets, void *d_ws, size_t ws_bytes, void *stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    const int G = group_blocks;
    if (dtype != PCX_F16 && dtype != PCX_BF16) PCX_FAIL(PCX_E_DTYPE, "pcx_mvmr_planned: fp16 or bf16 only (dtype %d)", dtype);
    if (C <= 0 || M <= 0 || n_feat < 0) PCX_FAIL(PCX_E_ARG, "pcx_mvmr_planned: bad sizes");
    if (!plan_sizes_ok(T, n_out, K, G))
        PCX_FAIL(PCX_E_UNSUPPORTED, "pcx_mvmr_planned: sizes out of range (T=%lld n_out=%lld K=%d group=%d)", (long long)T,
                 (long long)n_out, K, G);
    const int inw = transpose ? M : C, outw = transpose ? C : M;
    if (inw % 16 || outw % 16 || inw > 1024 || outw > 256)
        PCX_FAIL(PCX_E_UNSUPPORTED, "pcx_mvmr_planned: channel counts must be multiples of 16, output width at most 256 (C=%d M=%d)", C, M);
    if (!d_weight || !d_plan || !d_out || (T > 0 && !d_feat)) PCX_FAIL(PCX_E_ARG, "pcx_mvmr_planned: null pointer");
    if ((uintptr_t)d_weight % 16 || (uintptr_t)d_feat % 16 || (uintptr_t)d_out % 16 || (uintptr_t)d_plan % 256 || (uintptr_t)d_ws % 256)
        PCX_FAIL(PCX_E_ALIGN, "pcx_mvmr_planned: weight, features and output must be 16-byte aligned, plan and workspace 256-byte aligned");
    if (multi_buckets < 0 || multi_buckets > T / 2) PCX_FAIL(PCX_E_ARG, "pcx_mvmr_planned: multi_buckets out of range");
    if (multi_buckets > 0 && (!d_ws || ws_bytes < pcx_mvmr_planned_workspace_bytes(multi_buckets, transpose ? M : C)))
        PCX_FAIL(PCX_E_CAPACITY, "pcx_mvmr_planned: workspace %zu < %zu bytes", ws_bytes,
                 pcx_mvmr_planned_workspace_bytes(multi_buckets, transpose ? M : C));
    PlanView pv;
    const size_t need_plan = carve_plan(d_plan, T, n_out, K, G, &pv);
    if (plan_bytes < need_plan) PCX_FAIL(PCX_E_CAPACITY, "pcx_mvmr_planned: plan buffer %zu < %zu bytes", plan_bytes, need_plan);

    OsParams p = {};
    p.feat = (const uint16_t *)d_feat, p.out = (uint16_t *)d_out, p.weight = (const uint16_t *)d_weight;
    p.perm = pv.perm, p.tile_offs = pv.tile_offs, p.group_order = pv.group_order, p.entries = pv.entries, p.ctrl = pv.ctrl;
    p.tile_rows = pv.tile_rows, p.scratch = (const uint16_t *)d_ws;
    p.status = status_word();
    if (!p.status) PCX_FAIL(PCX_E_LAUNCH, "pcx_mvmr_planned: no device status word");
    p.K = K, p.C = C, p.M = M, p.transpose = transpose ? 1 : 0, p.fmt = dtype == PCX_BF16 ? 1 : 0;
    p.inw = inw, p.outw = outw, p.nkb = (inw + 63) / 64, p.G = G;
    p.ngroups = (int)pv.ngroups, p.nblocks = (int)pv.nblocks;
    p.col_stride = (uint32_t)((outw + 31) / 32 * 32);
    if ((uint32_t)G * p.col_stride > 512u)
        PCX_FAIL(PCX_E_UNSUPPORTED, "pcx_mvmr_planned: %d blocks of %d columns exceed the 512 TMEM columns", G, (int)p.col_stride);
    p.ncols = 32;
    while (p.ncols < (uint32_t)G * p.col_stride) p.ncols <<= 1;
    p.w_box_rows = (uint32_t)(transpose ? C : std::min(64, C));
    const uint32_t w_image = transpose ? (uint32_t)C * 128u : (uint32_t)((M + 63) / 64) * p.w_box_rows * 128u;
    p.w_slot_bytes = (uint32_t)align_up(w_image, 1024);
    p.w_tx_bytes = w_image;
    p.wait_limit_ns = wait_limit();
    p.use_tma = (M % 64 == 0) && encode_tiled() != nullptr;
    if (const char *e = getenv("PCX_OS_WTMA")) p.use_tma = p.use_tma && atoi(e) != 0;

    CUtensorMap tmap;
    memset(&tmap, 0, sizeof(tmap));
    if (p.use_tma) {
        const cuuint64_t gdim[2] = {(cuuint64_t)M, (cuuint64_t)K * (cuuint64_t)C};
        const cuuint64_t gstride[1] = {(cuuint64_t)M * 2};
        const cuuint32_t box[2] = {64u, p.w_box_rows};
        const cuuint32_t estride[2] = {1u, 1u};
        const CUresult r = encode_tiled()(&tmap, dtype == PCX_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                                          2, const_cast<void *>(d_weight), gdim, gstride, box, estride,
                                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) PCX_FAIL(PCX_E_LAUNCH, "pcx_mvmr_planned: cuTensorMapEncodeTiled failed (%d)", (int)r);
    }

    // Two CTAs share an SM when their accumulators fit half of the tensor memory: while one
    // writes its output rows or sets up its next group, the other keeps the tensor core and the
    // gathers going, and two threads issue MMAs.  Shared memory per CTA: A slots, weight slots,
    // the group's task tables.
    int ctas = p.ncols <= 256 ? 2 : 1;
    if (const char *e = getenv("PCX_OS_CTAS")) ctas = (atoi(e) == 1 || p.ncols > 256) ? 1 : 2;
    const size_t nkb = (size_t)p.nkb;
    const size_t table_fixed = align_up((size_t)G * K * nkb * 16 + ((size_t)G * K * 3 + 1 + (size_t)K * nkb) * 4, 16);
    const size_t static_smem = 512;
    int nslots = 0, nw = 0;
    for (; ctas >= 1 && !nslots; --ctas) {
        const size_t budget = (size_t)232448 / ctas - 1024 - static_smem - 1024;
        for (int a = MAX_SLOTS; a >= SIGNAL_LAG + 2 && !nslots; --a)
            for (int b = (ctas == 2 ? 3 : MAX_NW); b >= 2 && !nslots; --b)
                if ((size_t)a * SLOT_BYTES + (size_t)b * p.w_slot_bytes + table_fixed <= budget) nslots = a, nw = b;
        if (nslots) break;
    }
    if (!nslots) PCX_FAIL(PCX_E_UNSUPPORTED, "pcx_mvmr_planned: shared memory does not fit (K=%d C=%d M=%d group=%d)", K, C, M, G);
    int npw = MAX_NPW;
    if (const char *e = getenv("PCX_OS_WARPS")) {
        const int want = atoi(e);
        if (want == 4 || want == 8) npw = want;
    }
    if (const char *e = getenv("PCX_OS_SLOTS")) {
        const int want = atoi(e);
        if (want >= SIGNAL_LAG + 2 && want <= nslots) nslots = want;
    }
    if (const char *e = getenv("PCX_OS_WSLOTS")) {
        const int want = atoi(e);
        if (want >= 2 && want <= nw) nw = want;
    }
    p.npw = npw, p.nslots = nslots, p.nw = nw;
    p.lag = 0;
    if (const char *e = getenv("PCX_OS_LAG")) p.lag = atoi(e) ? SIGNAL_LAG : 0;
    const size_t smem = 1024 + (size_t)nslots * SLOT_BYTES + (size_t)nw * p.w_slot_bytes + table_fixed;
    static int granted[64] = {};
    int dev = 0;
    PCX_CUDA(cudaGetDevice(&dev));
    if ((int)smem > granted[dev & 63]) {
        PCX_CUDA(cudaFuncSetAttribute(mvmr_os_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        PCX_CUDA(cudaFuncSetAttribute(mvmr_os_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
        granted[dev & 63] = (int)smem;
    }
    const unsigned grid = (unsigned)std::max<int64_t>(1, std::min<int64_t>(pv.ngroups, (int64_t)ctas * num_sms()));
    if (multi_buckets > 0) {
        prof_begin("bucket_sum_kernel", stream);
        if (p.fmt) launch_bucket_sum<1>(multi_buckets, inw, p.feat, pv.entries, pv.buckets, pv.ctrl, (uint16_t *)d_ws, stream);
        else launch_bucket_sum<0>(multi_buckets, inw, p.feat, pv.entries, pv.buckets, pv.ctrl, (uint16_t *)d_ws, stream);
        prof_end(stream);
        PCX_LAUNCH_CHECK();
    }
    prof_begin(transpose ? "mvmr_os_kernel(dgrad)" : "mvmr_os_kernel(fwd)", stream);
    mvmr_os_kernel<<<grid, (unsigned)(npw + 2) * 32, smem, stream>>>(tmap, p);
    prof_end(stream);
    PCX_LAUNCH_CHECK();
    return PCX_OK;
}

int pcx_debug_wait_runs_out(unsigned long long limit_ns, void *stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    if (limit_ns == 0 || limit_ns > 100000000ull) PCX_FAIL(PCX_E_ARG, "pcx_debug_wait_runs_out: limit must be within (0, 100 ms]");
    unsigned int *status = status_word();
    if (!status) PCX_FAIL(PCX_E_LAUNCH, "pcx_debug_wait_runs_out: no device status word");
    wait_runs_out_kernel<<<1, 32, 0, stream>>>(status, 8u, (uint64_t)limit_ns);
    PCX_LAUNCH_CHECK();
    return PCX_OK;
}

}  // extern "C"
