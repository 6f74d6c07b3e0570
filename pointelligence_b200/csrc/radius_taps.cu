// Tap-segmented fixed-radius search in one enqueue and one host hand-over (sm_100a).
//
// Same result as pcx_radius_count + pcx_radius_fill with kernel_size > 0 -- the accepted
// (query i, point j) pairs grouped by kernel tap, inside a tap ordered by query, then by candidate
// cell, then by point index (internals/neighbors.py:469-838 followed by the stable sort by tap of
// layers/triplets.py:431-520) -- but built for latency instead of generality:
//
//   * points are binned by a HASH of their cell (side 2R), not by an injective key, so no extent
//     pass and no key-range hand-over precede the radix sort, and the bucket of a cell is found
//     with one load from a direct table.  Two cells may share a bucket: the foreign points are
//     ordinary candidates that fail the radius predicate (or the sample check), and the points of
//     the right cell keep their relative order (the sort is stable), so the output does not change.
//     The low three bits of the hash are the parities of the cell coordinates, so the eight cells
//     a query looks at always land in eight different buckets.
//   * eight lanes serve one query, one lane per candidate cell, each walking its own short run;
//     a block of 256 threads serves 32 consecutive queries.  The predicate runs alone over 64
//     candidates at a time into a bit mask; the rarer accepted points are handled afterwards, and
//     the fill pass reads the mask back instead of evaluating the predicate again.
//   * the count pass leaves a per-block tap histogram; its prefix over blocks plus the tap
//     segment offsets give every block its write position in every tap, so the fill pass places
//     the pairs directly in tap-major order (a stable counting sort by tap inside the block):
//     no sort of the edges, no per-query offsets.
//   * the fill pass writes into caller buffers of a given capacity; when the total exceeds it,
//     nothing is written and the call reports PCX_E_CAPACITY with the total, so that the caller
//     can retry with the exact size from the state kept in the workspace.
#include <cub/block/block_scan.cuh>
#include <cub/device/device_radix_sort.cuh>

#include <cfloat>
#include <cmath>

#include "geometry.cuh"

namespace pcx {
int device_status_address(unsigned int **d_status);   // status word of the bounded waits (sparse_tc.cu)
using namespace geo;
namespace {

constexpr int QPB = 32;           // queries per block
constexpr int THREADS = QPB * 8;  // one lane per (query, candidate cell)
constexpr int MAX_K3 = 128;       // taps this path handles (kernel_size 3 and 5)
constexpr int REC_MAX = 2048;     // accepted pairs staged per round of the fill pass
constexpr int SCAN_THREADS = 1024, SCAN_ITEMS = 4;

struct TapsWs {
    uint32_t *keys_a, *keys_b;
    int32_t *vals_a, *vals_b;
    float4 *sorted_pts;     // xyz + original index (bit pattern) in bucket order
    int2 *table;            // bucket -> [start, end) in the sorted order; (0,0) = empty
    uint4 *lanes;           // Q x 8: candidate run [start, end) and the accept mask of its first 64 points
    unsigned long long *lanes_more;   // Q x 8: accept mask of points 64 .. 127 of a run longer than 64
    uint32_t *lane_counts;  // Q x 8 accepted pairs per (query, cell)
    uint32_t *block_hist;   // [tap][block] accepted pairs; exclusive prefix over blocks after the scan
    unsigned long long *tap_total;  // k3
    int64_t *seg;           // k3 + 1
    int64_t *ctrl;          // [0] total pairs, [1] a tap's count does not fit 31 bits, [2] taps scanned,
                            // [3] queries without a neighbour
    void *cub_tmp;
    size_t cub_bytes;
    int bits;
    int64_t buckets, nblocks;
};

int bucket_bits(int64_t P) {
    int b = 1;
    while (((int64_t)1 << b) < P) ++b;
    b += 1;
    return b < 8 ? 8 : (b > 28 ? 28 : b);
}

size_t carve_taps(void *ws, int64_t P, int64_t Q, int k3, TapsWs *out) {
    Carver c(ws);
    TapsWs w;
    w.bits = bucket_bits(P);
    w.buckets = (int64_t)1 << w.bits;
    w.nblocks = (Q + QPB - 1) / QPB;
    w.ctrl = c.take<int64_t>(8);
    w.tap_total = c.take<unsigned long long>(k3);
    w.seg = c.take<int64_t>(k3 + 1);
    w.keys_a = c.take<uint32_t>(P);
    w.keys_b = c.take<uint32_t>(P);
    w.vals_a = c.take<int32_t>(P);
    w.vals_b = c.take<int32_t>(P);
    w.sorted_pts = c.take<float4>(P);
    w.table = c.take<int2>(w.buckets);
    w.lanes = c.take<uint4>(Q * 8);
    w.lanes_more = c.take<unsigned long long>(Q * 8);
    w.lane_counts = c.take<uint32_t>(Q * 8);
    w.block_hist = c.take<uint32_t>(w.nblocks * k3);
    w.cub_bytes = 0;
    cub::DeviceRadixSort::SortPairs(nullptr, w.cub_bytes, (const uint32_t *)nullptr, (uint32_t *)nullptr,
                                    (const int32_t *)nullptr, (int32_t *)nullptr, P);
    w.cub_tmp = c.take<char>(w.cub_bytes);
    if (out) *out = w;
    return c.off;
}

__device__ __forceinline__ uint32_t cell_bucket(int b, int cx, int cy, int cz, uint32_t mask) {
    uint32_t h = (uint32_t)(cx >> 1) * 73856093u ^ (uint32_t)(cy >> 1) * 19349663u ^ (uint32_t)(cz >> 1) * 83492791u ^
                 (uint32_t)b * 0x9E3779B1u;
    h ^= h >> 16, h *= 0x85ebca6bu, h ^= h >> 13, h *= 0xc2b2ae35u, h ^= h >> 16;
    return ((h << 3) | ((uint32_t)(cx & 1) << 2) | ((uint32_t)(cy & 1) << 1) | (uint32_t)(cz & 1)) & mask;
}

__global__ void taps_key_kernel(const float *__restrict__ pts, const int32_t *__restrict__ sample, int64_t P,
                                float inv, uint32_t mask, uint32_t *keys, int32_t *vals) {
    const int64_t p = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
    if (p >= P) return;
    keys[p] = cell_bucket(sample ? sample[p] : 0, cell_of(pts[3 * p], inv), cell_of(pts[3 * p + 1], inv),
                          cell_of(pts[3 * p + 2], inv), mask);
    vals[p] = (int32_t)p;
}

// Sorted copy of the points and the bucket table in one pass over the sorted keys.
__global__ void taps_table_kernel(const float *__restrict__ pts, const uint32_t *__restrict__ keys,
                                  const int32_t *__restrict__ perm, int64_t P, float4 *sorted_pts, int2 *table) {
    const int64_t s = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
    if (s >= P) return;
    const int32_t p = perm[s];
    sorted_pts[s] = make_float4(pts[3 * (int64_t)p], pts[3 * (int64_t)p + 1], pts[3 * (int64_t)p + 2], __int_as_float(p));
    const uint32_t key = keys[s];
    if (s == 0 || keys[s - 1] != key) table[key].x = (int)s;
    if (s + 1 == P || keys[s + 1] != key) table[key].y = (int)(s + 1);
}

struct TapArgs {
    const float *queries;
    const int32_t *query_sample, *point_sample;
    const float4 *sorted_pts;
    const int2 *table;
    uint4 *lanes;
    unsigned long long *lanes_more;
    uint32_t *lane_counts, *block_hist;
    int64_t *num_neighbors;
    const int64_t *seg, *ctrl;
    int64_t *ctrl_rw;
    int32_t *out_i, *out_j, *out_k;
    int64_t Q, nblocks, capacity;
    uint32_t mask;
    float r32, inv, g32, inv_g, s_max;
    int distance_type, variant, K, k3, use_s_max;
};

// The radius predicate without the square root where that is exact: sqrt is monotonic and correctly
// rounded, so sqrt(s) <= R holds exactly for the sums s up to the largest float whose root is <= R
// (s_max, found on the host).  The approximate-root variant and the Chebyshev distance keep the
// shared expression.
__device__ __forceinline__ bool accept_fast(const TapArgs &a, float qx, float qy, float qz, float4 p) {
    if (a.use_s_max) {
        const float dx = __fsub_rn(qx, p.x), dy = __fsub_rn(qy, p.y), dz = __fsub_rn(qz, p.z);
        const float s = a.variant == 0 ? __fadd_rn(__fadd_rn(__fmul_rn(dx, dx), __fmul_rn(dy, dy)), __fmul_rn(dz, dz))
                                       : __fmaf_rn(dz, dz, __fmaf_rn(dx, dx, __fmul_rn(dy, dy)));
        return s <= a.s_max;
    }
    float d;
    return radius_accept(qx, qy, qz, p, a.r32, a.distance_type, a.variant, &d);
}

// Walks the run [r.x, r.y) of sorted points for query (qx, qy, qz) of sample b, 64 candidates at a
// time: first the predicate alone over the chunk (two loads in flight, no divergent work), giving
// a 64-bit mask, then hit(tap, j) for the set bits in run order.  The mask of the first chunk is
// stored by the count pass (after the sample check) and read back by the fill pass, which then
// touches accepted points only; later chunks of a long run are evaluated again.  `masks` holds the
// masks of the first two chunks (128 candidates), which covers the runs of dense scenes.
template <bool STORED, typename Hit>
__device__ __forceinline__ void walk_run(const TapArgs &a, int2 r, float qx, float qy, float qz, int b,
                                         unsigned long long (&masks)[2], Hit hit) {
    for (int s0 = r.x; s0 < r.y; s0 += 64) {
        const int chunk = (s0 - r.x) >> 6;
        const bool first = chunk < 2;   // a chunk whose mask is kept
        const int len = min(64, r.y - s0);
        unsigned long long m = 0;
        if (STORED && first) {
            m = masks[chunk & 1];
        } else {
            uint32_t half[2] = {0u, 0u};
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int n = min(32, len - 32 * h);   // candidates of this half (may be <= 0)
                const float4 *src = a.sorted_pts + s0 + 32 * h;
                for (int t = 0; t < n; t += 4) {       // four loads in flight; the tail repeats the last point
                    float4 p[4];
#pragma unroll
                    for (int u = 0; u < 4; ++u) p[u] = src[min(t + u, n - 1)];
#pragma unroll
                    for (int u = 0; u < 4; ++u)
                        if (t + u < n && accept_fast(a, qx, qy, qz, p[u])) half[h] |= 1u << (t + u);
                }
            }
            m = (unsigned long long)half[0] | ((unsigned long long)half[1] << 32);
        }
        unsigned long long keep = m;
        while (m) {
            const int t = __ffsll((long long)m) - 1;
            m &= m - 1;
            const float4 p = a.sorted_pts[s0 + t];
            const int j = __float_as_int(p.w);
            if (!(STORED && first) && a.point_sample && a.point_sample[j] != b) {   // a foreign cell sharing the bucket
                keep &= ~(1ULL << t);
                continue;
            }
            hit(tap_of_fast(qx, qy, qz, p, a.g32, a.inv_g, a.K), j);
        }
        if (!STORED && first) masks[chunk & 1] = keep;
    }
}

__global__ void __launch_bounds__(THREADS) taps_count_kernel(TapArgs a) {
    __shared__ uint32_t s_hist[MAX_K3];
    if (threadIdx.x < MAX_K3) s_hist[threadIdx.x] = 0;
    __syncthreads();
    const int c = threadIdx.x & 7;
    const int64_t q = (int64_t)blockIdx.x * QPB + (threadIdx.x >> 3);
    uint32_t n = 0;
    if (q < a.Q) {
        const float qx = a.queries[3 * q], qy = a.queries[3 * q + 1], qz = a.queries[3 * q + 2];
        const int b = a.query_sample ? a.query_sample[q] : 0;
        const int cx = corner_of(qx, a.r32, a.inv) + ((c >> 2) & 1);
        const int cy = corner_of(qy, a.r32, a.inv) + ((c >> 1) & 1);
        const int cz = corner_of(qz, a.r32, a.inv) + (c & 1);
        const int2 r = a.table[cell_bucket(b, cx, cy, cz, a.mask)];
        unsigned long long masks[2] = {0ULL, 0ULL};
        walk_run<false>(a, r, qx, qy, qz, b, masks, [&](int tap, int) {
            ++n;
            atomicAdd(&s_hist[tap], 1u);
        });
        a.lanes[q * 8 + c] = make_uint4((uint32_t)r.x, (uint32_t)r.y, (uint32_t)masks[0], (uint32_t)(masks[0] >> 32));
        if (r.y - r.x > 64) a.lanes_more[q * 8 + c] = masks[1];
        a.lane_counts[q * 8 + c] = n;
    }
    uint32_t tot = n;
    tot += __shfl_xor_sync(0xffffffffu, tot, 1);
    tot += __shfl_xor_sync(0xffffffffu, tot, 2);
    tot += __shfl_xor_sync(0xffffffffu, tot, 4);
    if (q < a.Q && c == 0) {
        a.num_neighbors[q] = tot;
        if (tot == 0) atomicAdd((unsigned long long *)&a.ctrl_rw[3], 1ULL);
    }
    __syncthreads();
    if ((int)threadIdx.x < a.k3) a.block_hist[(int64_t)threadIdx.x * a.nblocks + blockIdx.x] = s_hist[threadIdx.x];
}

// One block per tap: exclusive prefix of the tap's counts over the query blocks (in place) and
// the tap's total; the block that finishes last turns the totals into the tap segment offsets.
__global__ void __launch_bounds__(SCAN_THREADS) taps_colscan_kernel(uint32_t *block_hist, int64_t nblocks, int k3,
                                                                     unsigned long long *tap_total, int64_t *seg,
                                                                     int64_t *seg_out, int64_t *ctrl) {
    using Scan = cub::BlockScan<uint32_t, SCAN_THREADS>;
    __shared__ typename Scan::TempStorage tmp;
    __shared__ int s_last;
    uint32_t *col = block_hist + (int64_t)blockIdx.x * nblocks;
    unsigned long long carry = 0;
    for (int64_t base = 0; base < nblocks; base += SCAN_THREADS * SCAN_ITEMS) {
        uint32_t v[SCAN_ITEMS], aggregate;
        const int64_t first = base + (int64_t)threadIdx.x * SCAN_ITEMS;
#pragma unroll
        for (int t = 0; t < SCAN_ITEMS; ++t) v[t] = first + t < nblocks ? col[first + t] : 0u;
        Scan(tmp).ExclusiveSum(v, v, aggregate);
#pragma unroll
        for (int t = 0; t < SCAN_ITEMS; ++t)
            if (first + t < nblocks) col[first + t] = (uint32_t)(carry + v[t]);
        carry += aggregate;
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        tap_total[blockIdx.x] = carry;
        if (carry > 0x7fffffffULL) ctrl[1] = 1;
        __threadfence();
        s_last = atomicAdd((unsigned long long *)&ctrl[2], 1ULL) == (unsigned long long)(k3 - 1);
    }
    __syncthreads();
    if (s_last && threadIdx.x < 32) {   // k3 <= 128: four taps per lane, prefix over the warp
        __threadfence();
        const int t0 = threadIdx.x * 4;
        unsigned long long v[4], sum = 0;
#pragma unroll
        for (int u = 0; u < 4; ++u) v[u] = t0 + u < k3 ? __ldcg(tap_total + t0 + u) : 0ULL, sum += v[u];
        unsigned long long incl = sum;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const unsigned long long up = __shfl_up_sync(0xffffffffu, incl, o);
            if ((int)threadIdx.x >= o) incl += up;
        }
        unsigned long long run = incl - sum;
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            if (t0 + u <= k3) seg[t0 + u] = (int64_t)run, seg_out[t0 + u] = (int64_t)run;
            run += v[u];
        }
        if (threadIdx.x == 31) ctrl[0] = (int64_t)incl, seg[k3] = (int64_t)incl, seg_out[k3] = (int64_t)incl;
    }
}

__global__ void __launch_bounds__(THREADS) taps_fill_kernel(TapArgs a) {
    using Scan = cub::BlockScan<uint32_t, THREADS>;
    const int kpad = (a.k3 + 31) & ~31;
    __shared__ typename Scan::TempStorage tmp;
    __shared__ unsigned long long s_rec[REC_MAX];   // tap << 40 | local query << 32 | point index, in output order
    extern __shared__ uint16_t s_gcnt[];            // [GROUPS][kpad] per 32 records and tap: count, then prefix inside the round
    __shared__ uint32_t s_base[MAX_K3];             // next write position of each tap for this block
    __shared__ uint32_t s_round[MAX_K3];
    if (a.ctrl[0] > a.capacity || a.ctrl[1]) return;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int c = threadIdx.x & 7, ql = threadIdx.x >> 3;
    const int64_t q0 = (int64_t)blockIdx.x * QPB, q = q0 + ql;
    if ((int)threadIdx.x < a.k3)
        s_base[threadIdx.x] = (uint32_t)a.seg[threadIdx.x] + a.block_hist[(int64_t)threadIdx.x * a.nblocks + blockIdx.x];
    const uint32_t n = q < a.Q ? a.lane_counts[q * 8 + c] : 0u;
    uint32_t my_off, block_total;
    Scan(tmp).ExclusiveSum(n, my_off, block_total);
    float qx = 0.f, qy = 0.f, qz = 0.f;
    int b = 0;
    int2 r = make_int2(0, 0);
    unsigned long long masks[2] = {0ULL, 0ULL};
    if (n) {
        qx = a.queries[3 * q], qy = a.queries[3 * q + 1], qz = a.queries[3 * q + 2];
        b = a.query_sample ? a.query_sample[q] : 0;
        const uint4 l = a.lanes[q * 8 + c];
        r = make_int2((int)l.x, (int)l.y);
        masks[0] = (unsigned long long)l.z | ((unsigned long long)l.w << 32);
        if (r.y - r.x > 64) masks[1] = a.lanes_more[q * 8 + c];
    }
    __syncthreads();
    for (uint32_t lo = 0; lo < block_total; lo += REC_MAX) {
        const uint32_t hi = lo + REC_MAX;
        const int cnt = (int)min((uint32_t)REC_MAX, block_total - lo), groups = (cnt + 31) >> 5;
        for (int t = threadIdx.x; t < groups * kpad; t += THREADS) s_gcnt[t] = 0;
        if (n && my_off < hi && my_off + n > lo) {
            uint32_t pos = my_off;
            walk_run<true>(a, r, qx, qy, qz, b, masks, [&](int tap, int j) {
                if (pos >= lo && pos < hi)
                    s_rec[pos - lo] = ((unsigned long long)tap << 40) | ((unsigned long long)ql << 32) | (uint32_t)j;
                ++pos;
            });
        }
        __syncthreads();
        // stable counting sort by tap: count per (32 records, tap), prefix over the groups, place
        for (int g = warp; g < groups; g += THREADS / 32) {
            const int idx = g * 32 + lane;
            const int tap = idx < cnt ? (int)(s_rec[idx] >> 40) : 0xffff;
            const unsigned m = __match_any_sync(0xffffffffu, tap);
            if (idx < cnt && lane == __ffs(m) - 1) s_gcnt[g * kpad + tap] = (uint16_t)__popc(m);
        }
        __syncthreads();
        if ((int)threadIdx.x < a.k3) {
            uint32_t run = 0;
            for (int g = 0; g < groups; ++g) {
                const uint32_t v = s_gcnt[g * kpad + threadIdx.x];
                s_gcnt[g * kpad + threadIdx.x] = (uint16_t)run;
                run += v;
            }
            s_round[threadIdx.x] = run;
        }
        __syncthreads();
        for (int g = warp; g < groups; g += THREADS / 32) {
            const int idx = g * 32 + lane;
            const unsigned long long rec = idx < cnt ? s_rec[idx] : ~0ULL;
            const int tap = idx < cnt ? (int)(rec >> 40) : 0xffff;
            const unsigned m = __match_any_sync(0xffffffffu, tap);
            if (idx < cnt) {
                const uint32_t pos = s_base[tap] + s_gcnt[g * kpad + tap] + __popc(m & ((1u << lane) - 1u));
                a.out_i[pos] = (int32_t)(q0 + (int)((rec >> 32) & 0xff));
                a.out_j[pos] = (int32_t)(uint32_t)rec;
                if (a.out_k) a.out_k[pos] = tap;
            }
        }
        __syncthreads();
        if ((int)threadIdx.x < a.k3) s_base[threadIdx.x] += s_round[threadIdx.x];
        __syncthreads();
    }
}

int check_common(int64_t P, int64_t Q, double radius, int distance_type, int kernel_size, double grid,
                 const char *who) {
    if (P <= 0 || Q <= 0) PCX_FAIL(PCX_E_ARG, "%s: P and Q must be positive (got %lld, %lld)", who, (long long)P, (long long)Q);
    if (P > INT32_MAX || Q > INT32_MAX) PCX_FAIL(PCX_E_UNSUPPORTED, "%s: more than 2^31-1 rows", who);
    if (!(radius > 0)) PCX_FAIL(PCX_E_ARG, "radius must be positive; got %g", radius);
    if (distance_type != 0 && distance_type != 1) PCX_FAIL(PCX_E_ARG, "distance_type must be 0 (ball) or 1 (chebyshev)");
    if (kernel_size <= 0 || kernel_size % 2 == 0) PCX_FAIL(PCX_E_ARG, "kernel_size must be a positive odd integer; got %d", kernel_size);
    if (kernel_size * kernel_size * kernel_size > MAX_K3)
        PCX_FAIL(PCX_E_UNSUPPORTED, "%s: kernel_size %d has more than %d taps; use pcx_radius_count / pcx_radius_fill", who, kernel_size, MAX_K3);
    if (!(grid > 0)) PCX_FAIL(PCX_E_ARG, "kernel_grid_size must be positive; got %g", grid);
    return PCX_OK;
}

TapArgs make_args(const TapsWs &w, const float *queries, const int32_t *point_sample, const int32_t *query_sample,
                  int64_t Q, double radius, int distance_type, int kernel_size, double grid) {
    TapArgs a = {};
    a.queries = queries, a.query_sample = query_sample, a.point_sample = point_sample;
    a.sorted_pts = w.sorted_pts, a.table = w.table, a.lanes = w.lanes, a.lanes_more = w.lanes_more;
    a.lane_counts = w.lane_counts, a.block_hist = w.block_hist, a.seg = w.seg, a.ctrl = w.ctrl, a.ctrl_rw = w.ctrl;
    a.Q = Q, a.nblocks = w.nblocks, a.mask = (uint32_t)(w.buckets - 1);
    a.r32 = (float)radius, a.inv = (float)(1.0 / (2.0 * radius)), a.g32 = (float)grid;
    a.inv_g = 1.0f / a.g32;
    a.distance_type = distance_type, a.variant = radius_variant(), a.K = kernel_size;
    a.k3 = kernel_size * kernel_size * kernel_size;
    a.use_s_max = distance_type == 0 && a.variant != 2;
    if (a.use_s_max) {   // largest float whose correctly rounded root is <= r32; r32 * r32 is within a few ulp of it
        float s = a.r32 * a.r32;
        if (!(s <= FLT_MAX)) s = FLT_MAX;
        for (int it = 0; it < 64 && s > 0.f && sqrtf(s) > a.r32; ++it) s = nextafterf(s, 0.f);
        for (int it = 0; it < 64 && s < FLT_MAX && sqrtf(nextafterf(s, FLT_MAX)) <= a.r32; ++it) s = nextafterf(s, FLT_MAX);
        a.use_s_max = sqrtf(s) <= a.r32 && (s == FLT_MAX || sqrtf(nextafterf(s, FLT_MAX)) > a.r32);
        a.s_max = s;
    }
    return a;
}

}  // namespace
}  // namespace pcx

using namespace pcx;

extern "C" {

int pcx_radius_taps_supported(int kernel_size) {
    return kernel_size > 0 && kernel_size % 2 == 1 && kernel_size * kernel_size * kernel_size <= MAX_K3;
}

size_t pcx_radius_taps_workspace_bytes(int64_t P, int64_t Q, int kernel_size) {
    if (P < 0 || Q < 0 || !pcx_radius_taps_supported(kernel_size)) return 0;
    return carve_taps(nullptr, P, Q, kernel_size * kernel_size * kernel_size, nullptr);
}

int pcx_radius_taps_count(const float *d_points, const float *d_queries, const int32_t *d_point_sample,
                          const int32_t *d_query_sample, int64_t P, int64_t Q, double radius, int distance_type,
                          int kernel_size, double kernel_grid_size, int64_t *d_num_neighbors, int64_t *d_seg_offs,
                          void *d_ws, size_t ws_bytes, void *stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    if (int rc = check_common(P, Q, radius, distance_type, kernel_size, kernel_grid_size, "pcx_radius_taps_count")) return rc;
    if (!d_points || !d_queries || !d_num_neighbors || !d_seg_offs || !d_ws) PCX_FAIL(PCX_E_ARG, "pcx_radius_taps_count: null pointer");
    if ((d_point_sample == nullptr) != (d_query_sample == nullptr)) PCX_FAIL(PCX_E_ARG, "pcx_radius_taps_count: sample ids must be given for both sets or neither");
    const int k3 = kernel_size * kernel_size * kernel_size;
    TapsWs w;
    const size_t need = carve_taps(d_ws, P, Q, k3, &w);
    if (ws_bytes < need) PCX_FAIL(PCX_E_CAPACITY, "pcx_radius_taps_count: workspace %zu < %zu bytes", ws_bytes, need);
    if ((uintptr_t)d_ws % 256) PCX_FAIL(PCX_E_ALIGN, "pcx_radius_taps_count: workspace must be 256-byte aligned");
    const float inv = (float)(1.0 / (2.0 * radius));
    const uint32_t mask = (uint32_t)(w.buckets - 1);
    const unsigned pblocks = (unsigned)((P + 255) / 256);
    PCX_CUDA(cudaMemsetAsync(w.ctrl, 0, 8 * sizeof(int64_t), stream));
    PCX_CUDA(cudaMemsetAsync(w.table, 0, (size_t)w.buckets * sizeof(int2), stream));
    taps_key_kernel<<<pblocks, 256, 0, stream>>>(d_points, d_point_sample, P, inv, mask, w.keys_a, w.vals_a);
    PCX_LAUNCH_CHECK();
    size_t tmp = w.cub_bytes;
    PCX_CUDA(cub::DeviceRadixSort::SortPairs(w.cub_tmp, tmp, w.keys_a, w.keys_b, w.vals_a, w.vals_b, P, 0, w.bits, stream));
    taps_table_kernel<<<pblocks, 256, 0, stream>>>(d_points, w.keys_b, w.vals_b, P, w.sorted_pts, w.table);
    PCX_LAUNCH_CHECK();
    TapArgs a = make_args(w, d_queries, d_point_sample, d_query_sample, Q, radius, distance_type, kernel_size, kernel_grid_size);
    a.num_neighbors = d_num_neighbors;
    prof_begin("taps_count_kernel", stream);
    taps_count_kernel<<<(unsigned)w.nblocks, THREADS, 0, stream>>>(a);
    prof_end(stream);
    PCX_LAUNCH_CHECK();
    taps_colscan_kernel<<<k3, SCAN_THREADS, 0, stream>>>(w.block_hist, w.nblocks, k3, w.tap_total, w.seg, d_seg_offs, w.ctrl);
    PCX_LAUNCH_CHECK();
    return PCX_OK;
}

int pcx_radius_taps_total(int64_t P, int64_t Q, int kernel_size, int64_t *h_total, void *d_ws, size_t ws_bytes,
                          void *stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    if (!h_total || !d_ws || P <= 0 || Q <= 0 || !pcx_radius_taps_supported(kernel_size)) PCX_FAIL(PCX_E_ARG, "pcx_radius_taps_total: bad arguments");
    TapsWs w;
    if (ws_bytes < carve_taps(d_ws, P, Q, kernel_size * kernel_size * kernel_size, &w)) PCX_FAIL(PCX_E_CAPACITY, "pcx_radius_taps_total: workspace too small");
    int64_t h[4] = {0, 0, 0, 0};
    unsigned int status = 0, *d_status = nullptr;
    if (int rc = device_status_address(&d_status)) return rc;
    PCX_CUDA(cudaMemcpyAsync(h, w.ctrl, sizeof(h), cudaMemcpyDeviceToHost, stream));
    PCX_CUDA(cudaMemcpyAsync(&status, d_status, sizeof(status), cudaMemcpyDeviceToHost, stream));
    PCX_CUDA(cudaStreamSynchronize(stream));
    h_total[0] = h[0], h_total[1] = h[3], h_total[2] = (int64_t)status;
    if (h[1] || h[0] > INT32_MAX) PCX_FAIL(PCX_E_UNSUPPORTED, "prepared kernel-segment output currently requires fewer than 2^31 edges; got %lld", (long long)h[0]);
    return PCX_OK;
}

int pcx_radius_taps_fill(const float *d_queries, const int32_t *d_point_sample, const int32_t *d_query_sample,
                         int64_t P, int64_t Q, double radius, int distance_type, int kernel_size,
                         double kernel_grid_size, int64_t capacity, int32_t *d_out_i, int32_t *d_out_j,
                         int32_t *d_out_k, int64_t *h_total, void *d_ws, size_t ws_bytes, void *stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    if (int rc = check_common(P, Q, radius, distance_type, kernel_size, kernel_grid_size, "pcx_radius_taps_fill")) return rc;
    if (!d_queries || !h_total || !d_ws || capacity < 0) PCX_FAIL(PCX_E_ARG, "pcx_radius_taps_fill: bad arguments");
    if (capacity > 0 && (!d_out_i || !d_out_j)) PCX_FAIL(PCX_E_ARG, "pcx_radius_taps_fill: d_out_i and d_out_j are required");
    if ((d_point_sample == nullptr) != (d_query_sample == nullptr)) PCX_FAIL(PCX_E_ARG, "pcx_radius_taps_fill: sample ids must be given for both sets or neither");
    const int k3 = kernel_size * kernel_size * kernel_size;
    TapsWs w;
    const size_t need = carve_taps(d_ws, P, Q, k3, &w);
    if (ws_bytes < need) PCX_FAIL(PCX_E_CAPACITY, "pcx_radius_taps_fill: workspace %zu < %zu bytes", ws_bytes, need);
    TapArgs a = make_args(w, d_queries, d_point_sample, d_query_sample, Q, radius, distance_type, kernel_size, kernel_grid_size);
    a.out_i = d_out_i, a.out_j = d_out_j, a.out_k = d_out_k, a.capacity = capacity;
    if (capacity > 0) {
        prof_begin("taps_fill_kernel", stream);
        taps_fill_kernel<<<(unsigned)w.nblocks, THREADS, (size_t)(REC_MAX / 32) * ((k3 + 31) & ~31) * sizeof(uint16_t), stream>>>(a);
        prof_end(stream);
        PCX_LAUNCH_CHECK();
    }
    int64_t h[4] = {0, 0, 0, 0};
    unsigned int status = 0, *d_status = nullptr;
    if (int rc = device_status_address(&d_status)) return rc;
    PCX_CUDA(cudaMemcpyAsync(h, w.ctrl, sizeof(h), cudaMemcpyDeviceToHost, stream));
    PCX_CUDA(cudaMemcpyAsync(&status, d_status, sizeof(status), cudaMemcpyDeviceToHost, stream));
    PCX_CUDA(cudaStreamSynchronize(stream));
    h_total[0] = h[0], h_total[1] = h[3], h_total[2] = (int64_t)status;
    if (h[1] || h[0] > INT32_MAX) PCX_FAIL(PCX_E_UNSUPPORTED, "prepared kernel-segment output currently requires fewer than 2^31 edges; got %lld", (long long)h[0]);
    if (h[0] > capacity) PCX_FAIL(PCX_E_CAPACITY, "pcx_radius_taps_fill: %lld pairs do not fit the capacity of %lld; nothing was written", (long long)h[0], (long long)capacity);
    return PCX_OK;
}

}  // extern "C"
