// Geometry stage of point convolution for sm_100a:
//   * exact fixed-radius search on a sorted grid of cell side 2R with optional
//     emission of the accepted pairs grouped by kernel tap;
//   * centre-nearest grid down-sampling.
//
// Both are integer/byte work bound by memory latency and HBM bandwidth: the
// points are binned with one 64-bit key each, sorted with a radix sort, and
// copied once into sorted float4 records so that the candidate scan of a
// query reads eight short contiguous runs.  One warp serves one query; lanes
// evaluate the predicate for 32 candidates at a time and compact the accepted
// ones with a ballot + popcount prefix, so the output order is deterministic.
//
// Arithmetic that decides membership is written with explicit round-to-nearest
// intrinsics (no FMA contraction) because the results have to be bit-identical
// with the reference:
//   cell of a point       floor(p * inv)            internals/neighbors.py:613-619
//   predicate             sqrt((dx^2+dy^2)+dz^2)<=R sparse_engines/strided_grid_radius_triton_kernel.py:25-31,127
//   tap                   rint((p-q) / g), clamped  sparse_engines/strided_grid_radius_triton_kernel.py:71-92
//   grid cell             Python-style floor div    internals/grid_indexing.py:20-27
//   centre distance       (dx^2+dy^2)+dz^2          internals/grid_sample_triton_kernel.py:68-104
#include <cub/device/device_radix_sort.cuh>
#include <cub/device/device_scan.cuh>

#include "geometry.cuh"

namespace pcx {
using namespace geo;
namespace {

constexpr int kWarpsPerBlock = 8;
constexpr int kSmemHistMax = 8192;  // taps kept in a shared-memory histogram

// ---------------------------------------------------------------- radius ----
struct RadiusWs {
    int32_t *ext;        // [0..2] min cell, [4..6] max cell, both over points and query corners
    int64_t *keys_a, *keys_b;
    int32_t *vals_a, *vals_b;
    float4 *sorted_pts;  // xyz + original index (bit pattern) in key order
    int32_t *sorted_sample;
    int2 *ranges;        // (start,end) of the 8 candidate cells per query
    int64_t *counts;     // Q+1, last entry 0
    int64_t *offsets;    // Q+1 exclusive scan, offsets[Q] = total
    uint32_t *tap_hist;  // K^3
    int64_t *seg;        // K^3+1 tap segment offsets (copy kept for the fill call)
    unsigned long long *max_key;  // largest cell key (bounds the radix sort's bit range)
    int64_t *cell_keys;  // open-addressing table: cell key -> (start,end) in the sorted order
    int2 *cell_ranges;
    int64_t cell_cap;    // table slots (power of two, at least 2 P)
    void *cub_tmp;
    size_t cub_bytes;
};

size_t radius_cub_bytes(int64_t P, int64_t Q) {
    size_t a = 0, b = 0;
    cub::DeviceRadixSort::SortPairs(nullptr, a, (const int64_t *)nullptr, (int64_t *)nullptr,
                                    (const int32_t *)nullptr, (int32_t *)nullptr, P);
    cub::DeviceScan::ExclusiveSum(nullptr, b, (const int64_t *)nullptr, (int64_t *)nullptr, Q + 1);
    return a > b ? a : b;
}

size_t carve_radius(void *ws, int64_t P, int64_t Q, int kernel_size, RadiusWs *out) {
    Carver c(ws);
    RadiusWs w;
    int64_t k3 = (int64_t)kernel_size * kernel_size * kernel_size;
    w.ext = c.take<int32_t>(8);
    w.keys_a = c.take<int64_t>(P);
    w.keys_b = c.take<int64_t>(P);
    w.vals_a = c.take<int32_t>(P);
    w.vals_b = c.take<int32_t>(P);
    w.sorted_pts = c.take<float4>(P);
    w.sorted_sample = c.take<int32_t>(P);
    w.ranges = c.take<int2>(Q * 8);
    w.counts = c.take<int64_t>(Q + 1);
    w.offsets = c.take<int64_t>(Q + 1);
    w.tap_hist = c.take<uint32_t>(k3 > 0 ? k3 : 1);
    w.seg = c.take<int64_t>(k3 + 1);
    w.max_key = c.take<unsigned long long>(1);
    w.cell_cap = 1024;
    while (w.cell_cap < 2 * P) w.cell_cap <<= 1;
    w.cell_keys = c.take<int64_t>(w.cell_cap);
    w.cell_ranges = c.take<int2>(w.cell_cap);
    w.cub_bytes = radius_cub_bytes(P, Q);
    w.cub_tmp = c.take<char>(w.cub_bytes);
    if (out) *out = w;
    return c.off;
}

// Running min / max of a thread's cells; folded per warp, then per block in shared memory, and
// only then into the global extents (one atomic per block and bound instead of one per warp).
struct Extent4 {
    int lo[4], hi[4];
    __device__ __forceinline__ void reset() {
#pragma unroll
        for (int a = 0; a < 4; ++a) lo[a] = INT_MAX, hi[a] = INT_MIN;
    }
    __device__ __forceinline__ void add(int a, int v) { lo[a] = min(lo[a], v), hi[a] = max(hi[a], v); }
};

__device__ __forceinline__ void block_minmax(Extent4 &e, int dims, int32_t *ext) {
    __shared__ int s_lo[4], s_hi[4];
    if (threadIdx.x < 4) s_lo[threadIdx.x] = INT_MAX, s_hi[threadIdx.x] = INT_MIN;
    __syncthreads();
    for (int a = 0; a < dims; ++a) {
        const int lo = __reduce_min_sync(0xffffffffu, e.lo[a]), hi = __reduce_max_sync(0xffffffffu, e.hi[a]);
        if ((threadIdx.x & 31) == 0) {
            if (lo != INT_MAX) atomicMin(&s_lo[a], lo);
            if (hi != INT_MIN) atomicMax(&s_hi[a], hi);
        }
    }
    __syncthreads();
    if ((int)threadIdx.x < dims) {
        if (s_lo[threadIdx.x] != INT_MAX) atomicMin(&ext[threadIdx.x], s_lo[threadIdx.x]);
        if (s_hi[threadIdx.x] != INT_MIN) atomicMax(&ext[4 + threadIdx.x], s_hi[threadIdx.x]);
    }
}

__global__ void radius_extent_kernel(const float *__restrict__ pts, const float *__restrict__ qry,
                                     int64_t P, int64_t Q, float inv, float r32, int32_t *ext) {
    const int64_t n = P + Q;
    Extent4 e;
    e.reset();
    for (int64_t t = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; t < n; t += (int64_t)gridDim.x * blockDim.x) {
        if (t < P) {
            e.add(0, cell_of(pts[3 * t], inv)), e.add(1, cell_of(pts[3 * t + 1], inv)), e.add(2, cell_of(pts[3 * t + 2], inv));
        } else {
            const int64_t q = t - P;
            e.add(0, corner_of(qry[3 * q], r32, inv)), e.add(1, corner_of(qry[3 * q + 1], r32, inv));
            e.add(2, corner_of(qry[3 * q + 2], r32, inv));
        }
    }
    block_minmax(e, 3, ext);
}

// Injective key of a cell of one sample.  Extents include the +1 candidate offset.
__device__ __forceinline__ int64_t cell_key(int b, int cx, int cy, int cz, const int32_t *ext) {
    int64_t ex = (int64_t)ext[4] - ext[0] + 2, ey = (int64_t)ext[5] - ext[1] + 2,
            ez = (int64_t)ext[6] - ext[2] + 2;
    return (((int64_t)b * ex + (cx - ext[0])) * ey + (cy - ext[1])) * ez + (cz - ext[2]);
}

__global__ void radius_key_kernel(const float *__restrict__ pts, const int32_t *__restrict__ sample,
                                  int64_t P, float inv, const int32_t *__restrict__ ext,
                                  int64_t *keys, int32_t *vals, unsigned long long *max_key) {
    int64_t p = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
    unsigned long long key = 0;
    if (p < P) {
        int b = sample ? sample[p] : 0;
        key = (unsigned long long)cell_key(b, cell_of(pts[3 * p], inv), cell_of(pts[3 * p + 1], inv),
                                           cell_of(pts[3 * p + 2], inv), ext);
        keys[p] = (int64_t)key;
        vals[p] = (int32_t)p;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) key = max(key, __shfl_xor_sync(0xffffffffu, key, o));
    if ((threadIdx.x & 31) == 0 && key) atomicMax(max_key, key);
}

// Cell table: key -> [start, end) of the cell's points in the sorted order.  Heads of
// runs insert (key, start); tails look their slot up and add the end.  Keys are >= 0.
constexpr int64_t CELL_EMPTY = -1;
__global__ void cell_table_heads_kernel(const int64_t *__restrict__ keys, int64_t P, int64_t *tkeys, int2 *tranges,
                                        uint64_t mask) {
    int64_t p = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
    if (p >= P) return;
    const int64_t key = keys[p];
    if (p > 0 && keys[p - 1] == key) return;
    uint64_t slot = mix64((uint64_t)key) & mask;
    for (;;) {   // the table is at most half full: an empty slot always turns up
        const long long prev = (long long)atomicCAS((unsigned long long *)&tkeys[slot], (unsigned long long)CELL_EMPTY,
                                                    (unsigned long long)key);
        if (prev == CELL_EMPTY) break;
        slot = (slot + 1) & mask;
    }
    tranges[slot].x = (int)p;
}
__device__ __forceinline__ int64_t cell_slot(const int64_t *__restrict__ tkeys, uint64_t mask, int64_t key) {
    uint64_t slot = mix64((uint64_t)key) & mask;
    for (;;) {
        const int64_t k = tkeys[slot];
        if (k == key) return (int64_t)slot;
        if (k == CELL_EMPTY) return -1;
        slot = (slot + 1) & mask;
    }
}
__global__ void cell_table_tails_kernel(const int64_t *__restrict__ keys, int64_t P, const int64_t *__restrict__ tkeys,
                                        int2 *tranges, uint64_t mask) {
    int64_t p = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
    if (p >= P) return;
    const int64_t key = keys[p];
    if (p + 1 < P && keys[p + 1] == key) return;
    const int64_t slot = cell_slot(tkeys, mask, key);
    if (slot >= 0) tranges[slot].y = (int)(p + 1);
}

__global__ void radius_gather_kernel(const float *__restrict__ pts, const int32_t *__restrict__ perm,
                                     int64_t P, float4 *sorted_pts) {
    int64_t s = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
    if (s >= P) return;
    int32_t p = perm[s];
    sorted_pts[s] = make_float4(pts[3 * (int64_t)p], pts[3 * (int64_t)p + 1], pts[3 * (int64_t)p + 2],
                                __int_as_float(p));
}

struct ScanArgs {
    const float *queries;
    const int32_t *query_sample;
    const float4 *sorted_pts;
    const int64_t *cell_keys;   // cell table (see cell_table_heads_kernel)
    const int2 *cell_ranges;
    uint64_t cell_mask;
    const int32_t *ext;
    int2 *ranges;
    int64_t P, Q;
    float r32, inv, g32;
    int distance_type, variant, K;
    // count outputs
    int64_t *counts;
    int64_t *num_neighbors;
    uint32_t *tap_hist;
    int use_smem_hist;
    // fill outputs
    const int64_t *offsets;
    int64_t *neighbors;
    float *distances;
    uint16_t *tap_keys;
    uint64_t *packed;
};

// MODE 0 = count, 1 = fill query-major neighbours, 2 = fill (tap, i, j) records
template <int MODE>
__global__ void __launch_bounds__(kWarpsPerBlock * 32) radius_scan_kernel(ScanArgs a) {
    extern __shared__ uint32_t s_hist[];
    const int lane = threadIdx.x & 31;
    const int k3 = a.K * a.K * a.K;
    if (MODE == 0 && a.K > 0 && a.use_smem_hist) {
        for (int t = threadIdx.x; t < k3; t += blockDim.x) s_hist[t] = 0;
        __syncthreads();
    }
    int64_t q = (int64_t)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
    if (q < a.Q) {
        float qx = a.queries[3 * q], qy = a.queries[3 * q + 1], qz = a.queries[3 * q + 2];
        int start = 0, end = 0;
        if (MODE == 0) {
            if (lane < 8) {
                int b = a.query_sample ? a.query_sample[q] : 0;
                int cx = corner_of(qx, a.r32, a.inv) + ((lane >> 2) & 1);
                int cy = corner_of(qy, a.r32, a.inv) + ((lane >> 1) & 1);
                int cz = corner_of(qz, a.r32, a.inv) + (lane & 1);
                const int64_t slot = cell_slot(a.cell_keys, a.cell_mask, cell_key(b, cx, cy, cz, a.ext));
                if (slot >= 0) {
                    const int2 r = a.cell_ranges[slot];
                    start = r.x, end = r.y;
                }
                a.ranges[q * 8 + lane] = make_int2(start, end);
            }
        } else if (lane < 8) {
            int2 r = a.ranges[q * 8 + lane];
            start = r.x, end = r.y;
        }
        int64_t out_base = MODE == 0 ? 0 : a.offsets[q];
        int found = 0;
        // The candidates of the 8 cells form one list (cell after cell, each in sorted order); the warp
        // walks it 64 at a time -- two independent loads per lane -- instead of one cell at a time, so
        // that half-empty cells cost no extra round trip to memory.
        int c_start[8], c_first[8];   // start of cell c in the sorted points, position of its first candidate in the list
        int total = 0;
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            const int s = __shfl_sync(0xffffffffu, start, c), e = __shfl_sync(0xffffffffu, end, c);
            c_start[c] = s, c_first[c] = total;
            total += e - s;
        }
        auto point_of = [&](int idx) {   // sorted-point index of list position idx
            int p = c_start[0] + idx;
#pragma unroll
            for (int c = 1; c < 8; ++c)
                if (idx >= c_first[c]) p = c_start[c] + (idx - c_first[c]);
            return p;
        };
        auto emit = [&](bool ok, float4 pt, float dist) {
            const unsigned m = __ballot_sync(0xffffffffu, ok);
            if (ok) {
                int tap = (a.K > 0) ? tap_of(qx, qy, qz, pt, a.g32, a.K) : 0;
                if (MODE == 0) {
                    if (a.K > 0) {
                        if (a.use_smem_hist) atomicAdd(&s_hist[tap], 1u);
                        else atomicAdd(&a.tap_hist[tap], 1u);
                    }
                } else {
                    int64_t pos = out_base + found + __popc(m & ((1u << lane) - 1u));
                    int32_t j = __float_as_int(pt.w);
                    if (MODE == 1) {
                        a.neighbors[pos] = j;
                        if (a.distances) a.distances[pos] = dist;
                    } else {
                        a.tap_keys[pos] = (uint16_t)tap;
                        a.packed[pos] = ((uint64_t)(uint32_t)q << 32) | (uint32_t)j;
                    }
                }
            }
            found += __popc(m);
        };
#pragma unroll 1
        for (int base = 0; base < total; base += 64) {
            const int i0 = base + lane, i1 = base + 32 + lane;
            float4 p0 = make_float4(0.f, 0.f, 0.f, 0.f), p1 = p0;
            if (i0 < total) p0 = a.sorted_pts[point_of(i0)];
            if (i1 < total) p1 = a.sorted_pts[point_of(i1)];
            float d0 = 0.f, d1 = 0.f;
            const bool ok0 = i0 < total && radius_accept(qx, qy, qz, p0, a.r32, a.distance_type, a.variant, &d0);
            const bool ok1 = i1 < total && radius_accept(qx, qy, qz, p1, a.r32, a.distance_type, a.variant, &d1);
            emit(ok0, p0, d0);
            if (base + 32 < total) emit(ok1, p1, d1);
        }
        if (MODE == 0 && lane == 0) {
            a.counts[q] = found;
            a.num_neighbors[q] = found;
        }
    }
    if (MODE == 0 && a.K > 0 && a.use_smem_hist) {
        __syncthreads();
        for (int t = threadIdx.x; t < k3; t += blockDim.x) {
            uint32_t v = s_hist[t];
            if (v) atomicAdd(&a.tap_hist[t], v);
        }
    }
}

__global__ void seg_offs_from_hist_kernel(const uint32_t *__restrict__ hist, int k3, int64_t *seg,
                                          int64_t *seg_copy) {
    // one thread; k3 is at most a few tens of thousands
    if (threadIdx.x == 0 && blockIdx.x == 0) {
        int64_t run = 0;
        for (int t = 0; t <= k3; ++t) {
            seg[t] = run;
            seg_copy[t] = run;
            if (t < k3) run += hist[t];
        }
    }
}

__global__ void unpack_pairs_kernel(const uint64_t *__restrict__ packed, int64_t T, int32_t *out_i,
                                    int32_t *out_j) {
    int64_t t = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
    if (t >= T) return;
    uint64_t v = packed[t];
    out_i[t] = (int32_t)(v >> 32);
    out_j[t] = (int32_t)(v & 0xffffffffu);
}

__global__ void set_last_zero_kernel(int64_t *counts, int64_t Q) { counts[Q] = 0; }

// -------------------------------------------------------- tap bookkeeping ----
__global__ void seg_offs_kernel(const int32_t *__restrict__ sorted, int64_t T, int K, int64_t *seg) {
    int k = blockIdx.x * blockDim.x + threadIdx.x;
    if (k > K) return;
    int64_t lo = 0, hi = T;
    while (lo < hi) {
        int64_t mid = (lo + hi) >> 1;
        if (sorted[mid] < k) lo = mid + 1; else hi = mid;
    }
    seg[k] = lo;
}

__global__ void expand_taps_kernel(const int64_t *__restrict__ seg, int K, int64_t T, int32_t *k_out) {
    int64_t t = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
    if (t >= T) return;
    int lo = 0, hi = K;  // largest k with seg[k] <= t
    while (hi - lo > 1) {
        int mid = (lo + hi) >> 1;
        if (seg[mid] <= t) lo = mid; else hi = mid;
    }
    k_out[t] = lo;
}

// ------------------------------------------------------------ grid sample ----
struct GridWs {
    int32_t *ext;  // min[4], max[4] of (x, y, z, sample)
    int64_t *keys_a, *keys_b;
    int32_t *vals_a, *vals_b;
    int32_t *flags;
    int32_t *ordinal;  // inclusive scan of flags
    void *cub_tmp;
    size_t cub_bytes;
};

size_t grid_cub_bytes(int64_t N) {
    size_t a = 0, b = 0;
    cub::DeviceRadixSort::SortPairs(nullptr, a, (const int64_t *)nullptr, (int64_t *)nullptr,
                                    (const int32_t *)nullptr, (int32_t *)nullptr, N);
    cub::DeviceScan::InclusiveSum(nullptr, b, (const int32_t *)nullptr, (int32_t *)nullptr, N);
    return a > b ? a : b;
}

size_t carve_grid(void *ws, int64_t N, GridWs *out) {
    Carver c(ws);
    GridWs w;
    w.ext = c.take<int32_t>(8);
    w.keys_a = c.take<int64_t>(N);
    w.keys_b = c.take<int64_t>(N);
    w.vals_a = c.take<int32_t>(N);
    w.vals_b = c.take<int32_t>(N);
    w.flags = c.take<int32_t>(N);
    w.ordinal = c.take<int32_t>(N);
    w.cub_bytes = grid_cub_bytes(N);
    w.cub_tmp = c.take<char>(w.cub_bytes);
    if (out) *out = w;
    return c.off;
}

// Python-style floor division of floats: the floor of the exact quotient a / b.
__device__ __forceinline__ int floor_div_cell(float a, float b) {
    float mod = fmodf(a, b);
    float div = __fdiv_rn(__fsub_rn(a, mod), b);
    if (mod != 0.f && ((b < 0.f) != (mod < 0.f))) div = __fsub_rn(div, 1.f);
    float fl;
    if (div != 0.f) {
        fl = floorf(div);
        if (__fsub_rn(div, fl) > 0.5f) fl = __fadd_rn(fl, 1.f);
    } else {
        fl = 0.f;
    }
    return (int)fl;
}

__global__ void grid_extent_kernel(const float *__restrict__ pts, const int32_t *__restrict__ sample,
                                   int64_t N, float cell, int32_t *ext) {
    Extent4 e;
    e.reset();
    for (int64_t t = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; t < N; t += (int64_t)gridDim.x * blockDim.x) {
        e.add(0, floor_div_cell(pts[3 * t], cell)), e.add(1, floor_div_cell(pts[3 * t + 1], cell));
        e.add(2, floor_div_cell(pts[3 * t + 2], cell));
        e.add(3, sample ? sample[t] : 0);
    }
    block_minmax(e, 4, ext);
}

__global__ void grid_key_kernel(const float *__restrict__ pts, const int32_t *__restrict__ sample,
                                int64_t N, float cell, const int32_t *__restrict__ ext,
                                int64_t *keys, int32_t *vals) {
    int64_t n = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
    if (n >= N) return;
    int64_t ex = (int64_t)ext[4] - ext[0] + 1, ey = (int64_t)ext[5] - ext[1] + 1,
            ez = (int64_t)ext[6] - ext[2] + 1;
    int64_t x = floor_div_cell(pts[3 * n], cell) - ext[0], y = floor_div_cell(pts[3 * n + 1], cell) - ext[1],
            z = floor_div_cell(pts[3 * n + 2], cell) - ext[2];
    int64_t b = (sample ? sample[n] : 0) - ext[3];
    keys[n] = x + ex * (y + ey * (z + ez * b));  // x fastest, sample slowest
    vals[n] = (int32_t)n;
}

__global__ void grid_flag_kernel(const int64_t *__restrict__ keys, int64_t N, int32_t *flags) {
    int64_t p = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
    if (p >= N) return;
    flags[p] = (p == 0 || keys[p] != keys[p - 1]) ? 1 : 0;
}

__global__ void grid_select_kernel(const float *__restrict__ pts, const int32_t *__restrict__ sample,
                                   const int64_t *__restrict__ keys, const int32_t *__restrict__ perm,
                                   const int32_t *__restrict__ flags, const int32_t *__restrict__ ordinal,
                                   int64_t N, float cell, int64_t *indices, float *out_pts,
                                   int32_t *out_sample, int64_t *mapping) {
    int64_t p = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
    if (p >= N) return;
    int32_t seg = ordinal[p] - 1;
    if (mapping) mapping[perm[p]] = seg;
    if (!flags[p]) return;
    int64_t key = keys[p];
    int32_t first = perm[p];
    float cx = __fmul_rn(__fadd_rn((float)floor_div_cell(pts[3 * (int64_t)first], cell), 0.5f), cell);
    float cy = __fmul_rn(__fadd_rn((float)floor_div_cell(pts[3 * (int64_t)first + 1], cell), 0.5f), cell);
    float cz = __fmul_rn(__fadd_rn((float)floor_div_cell(pts[3 * (int64_t)first + 2], cell), 0.5f), cell);
    float best = INFINITY;
    int32_t best_idx = first;
    for (int64_t r = p; r < N && keys[r] == key; ++r) {
        int32_t idx = perm[r];
        float dx = __fsub_rn(cx, pts[3 * (int64_t)idx]), dy = __fsub_rn(cy, pts[3 * (int64_t)idx + 1]),
              dz = __fsub_rn(cz, pts[3 * (int64_t)idx + 2]);
        float d2 = __fadd_rn(__fadd_rn(__fmul_rn(dx, dx), __fmul_rn(dy, dy)), __fmul_rn(dz, dz));
        if (d2 < best || (d2 == best && idx < best_idx)) {
            best = d2;
            best_idx = idx;
        }
    }
    indices[seg] = best_idx;
    out_pts[3 * (int64_t)seg] = pts[3 * (int64_t)best_idx];
    out_pts[3 * (int64_t)seg + 1] = pts[3 * (int64_t)best_idx + 1];
    out_pts[3 * (int64_t)seg + 2] = pts[3 * (int64_t)best_idx + 2];
    if (out_sample) out_sample[seg] = sample ? sample[best_idx] : 0;
}

int bits_for(int64_t n) {
    int b = 1;
    while (((int64_t)1 << b) < n) ++b;
    return b;
}

}  // namespace

// Predicate arithmetic in use (see radius_accept): 1 by default -- the FMA
// chain the reference's Triton kernels compile to on sm_100, measured on a B200
// -- overridable by the environment (PCX_RADIUS_PREDICATE) and at run time.
static std::atomic<int> g_radius_variant{-1};

int radius_variant() {
    int v = g_radius_variant.load();
    if (v < 0) {
        const char *e = getenv("PCX_RADIUS_PREDICATE");
        v = e ? atoi(e) : 1;
        if (v < 0 || v > 2) v = 1;
        g_radius_variant.store(v);
    }
    return v;
}

}  // namespace pcx

using namespace pcx;

extern "C" {

int pcx_set_radius_predicate(int variant) {
    if (variant < 0 || variant > 2) PCX_FAIL(PCX_E_ARG, "radius predicate variant must be 0, 1 or 2; got %d", variant);
    g_radius_variant.store(variant);
    return PCX_OK;
}

int pcx_get_radius_predicate(void) { return radius_variant(); }

size_t pcx_radius_workspace_bytes(int64_t P, int64_t Q, int kernel_size) {
    if (P < 0 || Q < 0 || kernel_size < 0) return 0;
    return carve_radius(nullptr, P, Q, kernel_size, nullptr);
}

size_t pcx_radius_fill_workspace_bytes(int64_t total, int kernel_size) {
    if (total <= 0 || kernel_size <= 0) return 256;
    Carver c(nullptr);
    c.take<uint16_t>(total);
    c.take<uint16_t>(total);
    c.take<uint64_t>(total);
    c.take<uint64_t>(total);
    size_t b = 0;
    cub::DeviceRadixSort::SortPairs(nullptr, b, (const uint16_t *)nullptr, (uint16_t *)nullptr,
                                    (const uint64_t *)nullptr, (uint64_t *)nullptr, total);
    c.take<char>(b);
    return c.off;
}

int pcx_radius_count(const float *d_points, const float *d_queries, const int32_t *d_point_sample,
                     const int32_t *d_query_sample, int64_t P, int64_t Q, double radius,
                     int distance_type, int kernel_size, double kernel_grid_size,
                     int64_t *d_num_neighbors, int64_t *d_seg_offs, int64_t *h_total, void *d_ws,
                     size_t ws_bytes, void *stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    if (P <= 0 || Q <= 0) PCX_FAIL(PCX_E_ARG, "pcx_radius_count: P and Q must be positive (got %lld, %lld)", (long long)P, (long long)Q);
    if (P > INT32_MAX || Q > INT32_MAX) PCX_FAIL(PCX_E_UNSUPPORTED, "pcx_radius_count: more than 2^31-1 rows");
    if (!d_points || !d_queries || !d_num_neighbors || !h_total || !d_ws) PCX_FAIL(PCX_E_ARG, "pcx_radius_count: null pointer");
    if ((d_point_sample == nullptr) != (d_query_sample == nullptr)) PCX_FAIL(PCX_E_ARG, "pcx_radius_count: sample ids must be given for both sets or neither");
    if (!(radius > 0)) PCX_FAIL(PCX_E_ARG, "radius must be positive; got %g", radius);
    if (distance_type != 0 && distance_type != 1) PCX_FAIL(PCX_E_ARG, "distance_type must be 0 (ball) or 1 (chebyshev)");
    if (kernel_size < 0 || (kernel_size > 0 && kernel_size % 2 == 0)) PCX_FAIL(PCX_E_ARG, "kernel_size must be a positive odd integer; got %d", kernel_size);
    if (kernel_size > 39) PCX_FAIL(PCX_E_UNSUPPORTED, "kernel_size above 39 is not supported");
    if (kernel_size > 0 && !(kernel_grid_size > 0)) PCX_FAIL(PCX_E_ARG, "kernel_grid_size must be positive; got %g", kernel_grid_size);
    if (kernel_size > 0 && !d_seg_offs) PCX_FAIL(PCX_E_ARG, "pcx_radius_count: d_seg_offs is required with kernel_size > 0");
    RadiusWs w;
    size_t need = carve_radius(d_ws, P, Q, kernel_size, &w);
    if (ws_bytes < need) PCX_FAIL(PCX_E_CAPACITY, "pcx_radius_count: workspace %zu < %zu bytes", ws_bytes, need);
    if ((uintptr_t)d_ws % 256) PCX_FAIL(PCX_E_ALIGN, "pcx_radius_count: workspace must be 256-byte aligned");

    const float r32 = (float)radius;
    const float inv = (float)(1.0 / (2.0 * radius));
    const int k3 = kernel_size * kernel_size * kernel_size;
    PCX_CUDA(cudaMemsetAsync(w.ext, 0x7f, 4 * sizeof(int32_t), stream));
    PCX_CUDA(cudaMemsetAsync(w.ext + 4, 0x80, 4 * sizeof(int32_t), stream));
    int blocks = (int)std::min<int64_t>((P + Q + 255) / 256, 8 * num_sms());
    radius_extent_kernel<<<blocks, 256, 0, stream>>>(d_points, d_queries, P, Q, inv, r32, w.ext);
    PCX_LAUNCH_CHECK();
    PCX_CUDA(cudaMemsetAsync(w.max_key, 0, sizeof(unsigned long long), stream));
    PCX_CUDA(cudaMemsetAsync(w.cell_keys, 0xff, (size_t)w.cell_cap * sizeof(int64_t), stream));
    radius_key_kernel<<<(unsigned)((P + 255) / 256), 256, 0, stream>>>(d_points, d_point_sample, P, inv, w.ext, w.keys_a, w.vals_a, w.max_key);
    PCX_LAUNCH_CHECK();
    // the sort only has to look at the bits the largest key uses (a hand-over of 8 bytes;
    // the call ends with one for the total anyway)
    unsigned long long h_max_key = 0;
    PCX_CUDA(cudaMemcpyAsync(&h_max_key, w.max_key, sizeof(h_max_key), cudaMemcpyDeviceToHost, stream));
    PCX_CUDA(cudaStreamSynchronize(stream));
    int key_bits = 1;
    while (key_bits < 64 && (h_max_key >> key_bits)) ++key_bits;
    size_t tmp = w.cub_bytes;
    PCX_CUDA(cub::DeviceRadixSort::SortPairs(w.cub_tmp, tmp, w.keys_a, w.keys_b, w.vals_a, w.vals_b, P, 0, key_bits, stream));
    radius_gather_kernel<<<(unsigned)((P + 255) / 256), 256, 0, stream>>>(d_points, w.vals_b, P, w.sorted_pts);
    PCX_LAUNCH_CHECK();
    const uint64_t cell_mask = (uint64_t)w.cell_cap - 1;
    cell_table_heads_kernel<<<(unsigned)((P + 255) / 256), 256, 0, stream>>>(w.keys_b, P, w.cell_keys, w.cell_ranges, cell_mask);
    PCX_LAUNCH_CHECK();
    cell_table_tails_kernel<<<(unsigned)((P + 255) / 256), 256, 0, stream>>>(w.keys_b, P, w.cell_keys, w.cell_ranges, cell_mask);
    PCX_LAUNCH_CHECK();
    if (k3 > 0) PCX_CUDA(cudaMemsetAsync(w.tap_hist, 0, (size_t)k3 * sizeof(uint32_t), stream));

    ScanArgs a = {};
    a.queries = d_queries, a.query_sample = d_query_sample, a.sorted_pts = w.sorted_pts;
    a.cell_keys = w.cell_keys, a.cell_ranges = w.cell_ranges, a.cell_mask = cell_mask;
    a.ext = w.ext, a.ranges = w.ranges, a.P = P, a.Q = Q;
    a.r32 = r32, a.inv = inv, a.g32 = (float)kernel_grid_size;
    a.distance_type = distance_type, a.variant = radius_variant(), a.K = kernel_size;
    a.counts = w.counts, a.num_neighbors = d_num_neighbors, a.tap_hist = w.tap_hist;
    a.use_smem_hist = (k3 > 0 && k3 <= kSmemHistMax) ? 1 : 0;
    size_t smem = a.use_smem_hist ? (size_t)k3 * sizeof(uint32_t) : 0;
    unsigned qblocks = (unsigned)((Q + kWarpsPerBlock - 1) / kWarpsPerBlock);
    radius_scan_kernel<0><<<qblocks, kWarpsPerBlock * 32, smem, stream>>>(a);
    PCX_LAUNCH_CHECK();
    set_last_zero_kernel<<<1, 1, 0, stream>>>(w.counts, Q);
    PCX_LAUNCH_CHECK();
    tmp = w.cub_bytes;
    PCX_CUDA(cub::DeviceScan::ExclusiveSum(w.cub_tmp, tmp, w.counts, w.offsets, Q + 1, stream));
    if (k3 > 0) {
        seg_offs_from_hist_kernel<<<1, 32, 0, stream>>>(w.tap_hist, k3, d_seg_offs, w.seg);
        PCX_LAUNCH_CHECK();
    }
    PCX_CUDA(cudaMemcpyAsync(h_total, w.offsets + Q, sizeof(int64_t), cudaMemcpyDeviceToHost, stream));
    PCX_CUDA(cudaStreamSynchronize(stream));
    return PCX_OK;
}

int pcx_radius_fill(const float *d_points, const float *d_queries, int64_t P, int64_t Q, double radius,
                    int distance_type, int kernel_size, double kernel_grid_size, int64_t total,
                    int64_t *d_neighbors, float *d_distances, int32_t *d_out_i, int32_t *d_out_j,
                    int32_t *d_out_k, void *d_ws, size_t ws_bytes, void *d_ws2, size_t ws2_bytes,
                    void *stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    (void)d_points;
    if (total == 0) return PCX_OK;
    if (P <= 0 || Q <= 0 || total < 0) PCX_FAIL(PCX_E_ARG, "pcx_radius_fill: bad sizes");
    if (!d_queries || !d_ws) PCX_FAIL(PCX_E_ARG, "pcx_radius_fill: null pointer");
    if (kernel_size == 0 && !d_neighbors) PCX_FAIL(PCX_E_ARG, "pcx_radius_fill: d_neighbors is required");
    if (kernel_size > 0 && (!d_out_i || !d_out_j || !d_ws2)) PCX_FAIL(PCX_E_ARG, "pcx_radius_fill: d_out_i, d_out_j and d_ws2 are required with kernel_size > 0");
    if (kernel_size > 0 && total > INT32_MAX) PCX_FAIL(PCX_E_UNSUPPORTED, "prepared kernel-segment output currently requires fewer than 2^31 edges; got %lld", (long long)total);
    RadiusWs w;
    size_t need = carve_radius(d_ws, P, Q, kernel_size, &w);
    if (ws_bytes < need) PCX_FAIL(PCX_E_CAPACITY, "pcx_radius_fill: workspace %zu < %zu bytes", ws_bytes, need);
    const int k3 = kernel_size * kernel_size * kernel_size;

    ScanArgs a = {};
    a.queries = d_queries, a.sorted_pts = w.sorted_pts, a.ext = w.ext;
    a.ranges = w.ranges, a.P = P, a.Q = Q;
    a.r32 = (float)radius, a.inv = (float)(1.0 / (2.0 * radius)), a.g32 = (float)kernel_grid_size;
    a.distance_type = distance_type, a.variant = radius_variant(), a.K = kernel_size;
    a.offsets = w.offsets;
    unsigned qblocks = (unsigned)((Q + kWarpsPerBlock - 1) / kWarpsPerBlock);
    if (kernel_size == 0) {
        a.neighbors = d_neighbors, a.distances = d_distances;
        radius_scan_kernel<1><<<qblocks, kWarpsPerBlock * 32, 0, stream>>>(a);
        PCX_LAUNCH_CHECK();
        return PCX_OK;
    }
    size_t need2 = pcx_radius_fill_workspace_bytes(total, kernel_size);
    if (ws2_bytes < need2) PCX_FAIL(PCX_E_CAPACITY, "pcx_radius_fill: fill workspace %zu < %zu bytes", ws2_bytes, need2);
    Carver c(d_ws2);
    uint16_t *key_a = c.take<uint16_t>(total), *key_b = c.take<uint16_t>(total);
    uint64_t *val_a = c.take<uint64_t>(total), *val_b = c.take<uint64_t>(total);
    size_t cub_bytes = 0;
    cub::DeviceRadixSort::SortPairs(nullptr, cub_bytes, (const uint16_t *)nullptr, (uint16_t *)nullptr,
                                    (const uint64_t *)nullptr, (uint64_t *)nullptr, total);
    void *cub_tmp = c.take<char>(cub_bytes);
    a.tap_keys = key_a, a.packed = val_a;
    radius_scan_kernel<2><<<qblocks, kWarpsPerBlock * 32, 0, stream>>>(a);
    PCX_LAUNCH_CHECK();
    const uint64_t *sorted_vals = val_a;
    if (k3 > 1) {
        PCX_CUDA(cub::DeviceRadixSort::SortPairs(cub_tmp, cub_bytes, key_a, key_b, val_a, val_b, total, 0,
                                                 bits_for(k3), stream));
        sorted_vals = val_b;
    }
    unpack_pairs_kernel<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(sorted_vals, total, d_out_i, d_out_j);
    PCX_LAUNCH_CHECK();
    if (d_out_k) {
        expand_taps_kernel<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(w.seg, k3, total, d_out_k);
        PCX_LAUNCH_CHECK();
    }
    return PCX_OK;
}

int pcx_seg_offs(const int32_t *d_sorted, int64_t T, int K, int64_t *d_seg_offs, void *stream) {
    if (K <= 0 || T < 0 || !d_seg_offs || (T > 0 && !d_sorted)) PCX_FAIL(PCX_E_ARG, "pcx_seg_offs: bad arguments");
    seg_offs_kernel<<<(K + 1 + 127) / 128, 128, 0, (cudaStream_t)stream>>>(d_sorted, T, K, d_seg_offs);
    PCX_LAUNCH_CHECK();
    return PCX_OK;
}

int pcx_expand_taps(const int64_t *d_seg_offs, int K, int64_t T, int32_t *d_k, void *stream) {
    if (K <= 0 || T < 0 || !d_seg_offs || (T > 0 && !d_k)) PCX_FAIL(PCX_E_ARG, "pcx_expand_taps: bad arguments");
    if (T == 0) return PCX_OK;
    expand_taps_kernel<<<(unsigned)((T + 255) / 256), 256, 0, (cudaStream_t)stream>>>(d_seg_offs, K, T, d_k);
    PCX_LAUNCH_CHECK();
    return PCX_OK;
}

size_t pcx_grid_sample_workspace_bytes(int64_t N) {
    if (N < 0) return 0;
    return carve_grid(nullptr, N, nullptr);
}

int pcx_grid_sample_count(const float *d_points, const int32_t *d_sample, int64_t N, double cell,
                          int64_t *h_num_cells, void *d_ws, size_t ws_bytes, void *stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    if (N <= 0 || !d_points || !h_num_cells || !d_ws) PCX_FAIL(PCX_E_ARG, "pcx_grid_sample_count: bad arguments");
    if (N > INT32_MAX) PCX_FAIL(PCX_E_UNSUPPORTED, "pcx_grid_sample_count: more than 2^31-1 points");
    if (!(cell > 0)) PCX_FAIL(PCX_E_ARG, "grid_size must be positive; got %g", cell);
    GridWs w;
    size_t need = carve_grid(d_ws, N, &w);
    if (ws_bytes < need) PCX_FAIL(PCX_E_CAPACITY, "pcx_grid_sample_count: workspace %zu < %zu bytes", ws_bytes, need);
    if ((uintptr_t)d_ws % 256) PCX_FAIL(PCX_E_ALIGN, "pcx_grid_sample_count: workspace must be 256-byte aligned");
    const float c32 = (float)cell;
    PCX_CUDA(cudaMemsetAsync(w.ext, 0x7f, 4 * sizeof(int32_t), stream));
    PCX_CUDA(cudaMemsetAsync(w.ext + 4, 0x80, 4 * sizeof(int32_t), stream));
    int blocks = (int)std::min<int64_t>((N + 255) / 256, 8 * num_sms());
    grid_extent_kernel<<<blocks, 256, 0, stream>>>(d_points, d_sample, N, c32, w.ext);
    PCX_LAUNCH_CHECK();
    unsigned nb = (unsigned)((N + 255) / 256);
    grid_key_kernel<<<nb, 256, 0, stream>>>(d_points, d_sample, N, c32, w.ext, w.keys_a, w.vals_a);
    PCX_LAUNCH_CHECK();
    // The sort only has to look at the bits the largest key can use: the extents come to the host
    // (32 bytes; the call ends with a hand-over of the cell count anyway).
    int32_t h_ext[8];
    PCX_CUDA(cudaMemcpyAsync(h_ext, w.ext, sizeof(h_ext), cudaMemcpyDeviceToHost, stream));
    PCX_CUDA(cudaStreamSynchronize(stream));
    int key_bits = 64;
    {
        uint64_t span = 1;
        bool fits = true;
        for (int a = 0; a < 4 && fits; ++a) {
            const int64_t e = (int64_t)h_ext[4 + a] - h_ext[a] + 1;
            fits = e > 0 && !__builtin_mul_overflow(span, (uint64_t)e, &span);
        }
        if (fits) {
            key_bits = 1;
            while (key_bits < 64 && ((span - 1) >> key_bits)) ++key_bits;
        }
    }
    size_t tmp = w.cub_bytes;
    PCX_CUDA(cub::DeviceRadixSort::SortPairs(w.cub_tmp, tmp, w.keys_a, w.keys_b, w.vals_a, w.vals_b, N, 0, key_bits, stream));
    grid_flag_kernel<<<nb, 256, 0, stream>>>(w.keys_b, N, w.flags);
    PCX_LAUNCH_CHECK();
    tmp = w.cub_bytes;
    PCX_CUDA(cub::DeviceScan::InclusiveSum(w.cub_tmp, tmp, w.flags, w.ordinal, N, stream));
    int32_t last = 0;
    PCX_CUDA(cudaMemcpyAsync(&last, w.ordinal + (N - 1), sizeof(int32_t), cudaMemcpyDeviceToHost, stream));
    PCX_CUDA(cudaStreamSynchronize(stream));
    *h_num_cells = last;
    return PCX_OK;
}

int pcx_grid_sample_select(const float *d_points, const int32_t *d_sample, int64_t N, double cell,
                           int64_t num_cells, int64_t *d_indices, float *d_out_points,
                           int32_t *d_out_sample, int64_t *d_mapping, void *d_ws, size_t ws_bytes,
                           void *stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    if (N <= 0 || num_cells <= 0 || !d_points || !d_indices || !d_out_points || !d_ws) PCX_FAIL(PCX_E_ARG, "pcx_grid_sample_select: bad arguments");
    GridWs w;
    size_t need = carve_grid(d_ws, N, &w);
    if (ws_bytes < need) PCX_FAIL(PCX_E_CAPACITY, "pcx_grid_sample_select: workspace %zu < %zu bytes", ws_bytes, need);
    grid_select_kernel<<<(unsigned)((N + 255) / 256), 256, 0, stream>>>(
        d_points, d_sample, w.keys_b, w.vals_b, w.flags, w.ordinal, N, (float)cell, d_indices,
        d_out_points, d_out_sample, d_mapping);
    PCX_LAUNCH_CHECK();
    return PCX_OK;
}

}  // extern "C"
