// Tensor-core engines for MVMR and VVOR on sm_100a (tcgen05 + TMEM).
//
// Both kernels are persistent: every CTA owns a contiguous range of chunks of
// 128 tap-sorted triplets.  A chunk is gathered row by row with 16-byte
// cp.async copies straight into the 128-byte-swizzled shared-memory layout the
// tensor core reads, so no separate staging pass exists:
//
//   smem tile  = [64-channel block][row][128 bytes], 16-byte pieces XOR-swizzled
//                with (row & 7)  (the SWIZZLE_128B canonical layout)
//
//   MVMR   D[128 triplets x N] = A[128 x Kc] * B[Kc x N]
//          A = gathered feature rows   (K-major: a row is contiguous along Kc)
//          B = W[tap] exactly as stored, (C, M) row-major: read MN-major in the
//              forward (its rows are the contraction index) and K-major in the
//              input gradient (its rows are the output channels)
//          one A tile per CTA; latency is hidden by the other CTAs resident on the
//          SM (5-6 at C = 64), so shared memory per CTA is kept as small as possible
//          epilogue, rows of 64 floats: TMEM -> registers -> a parking area in shared
//          memory (16 rows per warp at a time, aliased with the A tile) -> one bulk
//          reduction (cp.reduce.async.bulk add.f32) per output row;
//          other widths: TMEM -> registers -> red.global.add.v2.f32
//   VVOR   D[Ma x Cb] += X[t x Ma]^T * G[t x Cb], t = triplets of the chunk
//          both operands MN-major (a gathered row is contiguous along M / N,
//          the triplet index is the contraction), accumulated in TMEM over all
//          chunks of a tap and flushed once per (CTA, tap); one operand stage by
//          default (a ring of up to 4 is available)
//
// Measured on B200, both kernels are bound by latency, not by a pipe: at C = 64 the
// L2 runs at about a third of its throughput and DRAM at a tenth, and every step that
// put more CTAs on an SM (3 -> 5 -> 6) shortened the kernel (78 -> 64 -> 62 us).
//
// One thread issues tcgen05.mma; completion is signalled with tcgen05.commit on
// an mbarrier.  Every wait is bounded (one second): after the limit the kernel raises a flag
// in the status word, frees its TMEM and returns.
#include "sparse_kernels.cuh"
#include "tcgen05.cuh"

namespace pcx {

__device__ unsigned int g_device_status = 0;

namespace {

constexpr int CH = 128;            // triplets per chunk
constexpr int BLK_BYTES = CH * 128; // one 64-channel block of a 128-row tile

using namespace tc;

// Position of a CTA in the chunk sequence; the bounds of the current tap are
// kept in registers and reloaded only when the chunk index leaves the tap.
// The cumulative chunk table lives in shared memory (built by every CTA from
// the segment offsets), so no separate kernel and no global table are needed.
template <int CHR>
struct ChunkCursorT {
    int tap;
    int cum_lo, cum_hi;
    int64_t seg_lo, seg_hi;
    __device__ __forceinline__ void load(const int32_t *cum, const int64_t *__restrict__ seg) {
        cum_lo = cum[tap], cum_hi = cum[tap + 1];
        seg_lo = seg[tap], seg_hi = seg[tap + 1];
    }
    __device__ __forceinline__ void seek(const int32_t *cum, const int64_t *__restrict__ seg, int K, int chunk) {
        int lo = 0, hi = K;
        while (hi - lo > 1) {
            int mid = (lo + hi) >> 1;
            if (cum[mid] <= chunk) lo = mid; else hi = mid;
        }
        tap = lo;
        load(cum, seg);
    }
    __device__ __forceinline__ void advance(const int32_t *cum, const int64_t *__restrict__ seg, int K, int chunk) {
        if (chunk < cum_hi) return;
        while (tap + 1 < K && cum[tap + 1] <= chunk) ++tap;
        load(cum, seg);
    }
    __device__ __forceinline__ int64_t first(int chunk) const { return seg_lo + (int64_t)(chunk - cum_lo) * CHR; }
    __device__ __forceinline__ int rows(int chunk) const {
        int64_t left = seg_hi - first(chunk);
        return (int)(left < CHR ? left : CHR);
    }
    __device__ __forceinline__ bool last_of_tap(int chunk) const { return chunk + 1 >= cum_hi; }
};
using ChunkCursor = ChunkCursorT<CH>;

constexpr int MAX_TAPS_SMEM = 1024;  // taps whose chunk table fits the shared-memory copy

// cum[k] = chunks of CHR triplets in the taps before k; all threads of the CTA call this.
template <int CHR = CH>
__device__ __forceinline__ void build_chunk_table(const int64_t *__restrict__ seg, int K, int32_t *cum,
                                                  int32_t *warp_sums) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
    int32_t carry = 0;
    for (int base = 0; base < K; base += blockDim.x) {
        int k = base + tid;
        int32_t v = k < K ? (int32_t)((seg[k + 1] - seg[k] + CHR - 1) / CHR) : 0;
        int32_t inc = v;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            int32_t n = __shfl_up_sync(0xffffffffu, inc, o);
            if (lane >= o) inc += n;
        }
        if (lane == 31) warp_sums[warp] = inc;
        __syncthreads();
        int32_t before = carry, all = carry;
        for (int w = 0; w < nwarps; ++w) {
            if (w < warp) before += warp_sums[w];
            all += warp_sums[w];
        }
        if (k < K) cum[k] = before + inc - v;
        carry = all;
        __syncthreads();
    }
    if (tid == 0) cum[K] = carry;
    __syncthreads();
}

// Gather `rows` rows of `width` 2-byte channels into a swizzled tile; the row
// indices were staged in shared memory beforehand so that the copy loop issues
// cp.async back to back.  Rows past `rows` are zero-filled when ZERO_TAIL
// (needed when the row index is the contraction index), untouched otherwise.
template <bool ZERO_TAIL, int CHR = CH>
__device__ __forceinline__ void gather_tile(uint32_t tile, const uint16_t *__restrict__ src,
                                            const int32_t *s_idx, int rows, int width, int tid, int nthreads) {
    const int cpr = width >> 3;  // 16-byte pieces per row
    constexpr uint32_t BLK = CHR * 128;   // one 64-channel block of the tile
    const int rmax = ZERO_TAIL ? CHR : rows;
    if ((cpr & (cpr - 1)) == 0) {
        // power-of-two row length: a thread keeps its 16-byte column and walks down the rows
        const int sh = __ffs(cpr) - 1;
        const int ch = tid & (cpr - 1), rpp = nthreads >> sh;
        const uint32_t dcol = tile + (uint32_t)(ch >> 3) * BLK;
        const uint16_t *scol = src + ch * 8;
#pragma unroll 4
        for (int r = tid >> sh; r < rmax; r += rpp) {
            const uint32_t dst = dcol + (uint32_t)r * 128 + (uint32_t)(((ch ^ r) & 7) << 4);
            if (r < rows) {
                cp_async16(dst, scol + (int64_t)s_idx[r] * width);
            } else if (ZERO_TAIL) {
                asm volatile("st.shared.v4.b32 [%0], {%1,%1,%1,%1};" ::"r"(dst), "r"(0) : "memory");
            }
        }
        return;
    }
    // (keeping a thread on one column with a single division up front was tried for these row
    // lengths and for the loop above: 96 channels unchanged, 128 and 256 channels 13 % slower)
    for (int e = tid; e < rmax * cpr; e += nthreads) {
        int r = e / cpr, ch = e - r * cpr;
        uint32_t dst = tile + (uint32_t)(ch >> 3) * BLK + (uint32_t)r * 128 + (uint32_t)(((ch & 7) ^ (r & 7)) << 4);
        if (r < rows) {
            cp_async16(dst, src + (int64_t)s_idx[r] * width + ch * 8);
        } else if (ZERO_TAIL) {
            asm volatile("st.shared.v4.b32 [%0], {%1,%1,%1,%1};" ::"r"(dst), "r"(0) : "memory");
        }
    }
}

// Scatter through the copy engine: every accumulator row is parked in shared
// memory and handed to one bulk reduction (fp32 add into global memory), so the
// scatter neither occupies the load/store pipeline nor needs one instruction
// per 32-byte piece.
__device__ __forceinline__ void bulk_reduce_add_f32(float *gdst, uint32_t ssrc, uint32_t bytes) {
    asm volatile("cp.reduce.async.bulk.global.shared::cta.bulk_group.add.f32 [%0], [%1], %2;"
                 ::"l"(gdst), "r"(ssrc), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }


__device__ __forceinline__ uint32_t pack_pair(float a, float b, int fmt) {
    if (fmt) {
        __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
        return *reinterpret_cast<uint32_t *>(&h);
    }
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t *>(&h);
}

struct MvmrTcParams {
    const uint16_t *weight;  // (K, C, M) as stored
    const uint16_t *feat;
    const int32_t *gather, *scatter;
    const int64_t *seg;
    float *acc;
    uint16_t *out;           // MODE 2: the output rows themselves (every row occurs in exactly one triplet)
    int K, C, M, transpose, fmt, nbuf, slab;  // slab: columns parked per bulk reduction (32 or 64)
    int prow_log2;                            // a warp parks 2^prow_log2 rows at a time (8, 16 or 32)
    uint32_t park_bytes;                      // size of the parking area (the chunk table follows it)
    int alias;                                // parking area shares the feature tile's memory
    uint32_t ncols;
};

// One A tile by default: the next gather is issued as soon as the multiply has finished (or,
// when the parking area aliases the tile, once the reductions have read it) and the other
// CTAs resident on the SM cover its latency; the indices of chunk c+2 are already on their
// way into registers.  nbuf == 2 keeps a ring of two A tiles instead.
// MODE 0: sums leave through two-float reductions from registers; 1: one bulk reduction per row
// (rows of 64 floats); 2: plain 16-byte stores of the rounded row, for rulebooks in which every output
// row occurs in exactly one triplet (fan-in 1: nothing to accumulate, clear or round afterwards).
template <int MODE>
__global__ void __launch_bounds__(128) mvmr_tc_kernel(MvmrTcParams p) {
    constexpr bool BULK = MODE == 1;
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t s_bar;
    __shared__ uint32_t s_tmem;
    __shared__ __align__(16) int32_t s_scatter[2][CH];
    __shared__ int32_t s_gather[2][CH];
    __shared__ int32_t s_warp_sums[4];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int inw = p.transpose ? p.M : p.C, outw = p.transpose ? p.C : p.M;
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const int kb = (inw + 63) >> 6;
    const uint32_t a_bytes = (uint32_t)kb * BLK_BYTES;
    // layout: weight tile | feature tile(s) | parking area | chunk table; when the parking area
    // aliases the feature tile (p.alias) it starts where the feature tile starts
    const uint32_t b_tile = base;
    const uint32_t a_tile0 = b_tile + (uint32_t)((p.M + 63) >> 6) * (uint32_t)p.C * 128;
    const bool two = p.nbuf == 2;
    // the weight tile is W[tap] as stored: C rows of M channels, 64-channel blocks
    const uint32_t w_blk = (uint32_t)p.C * 128;
    const uint32_t bar = smem_u32(&s_bar);
    // per-warp parking area of the scatter: 32 rows of slab floats, rows padded by 16 bytes
    const uint32_t park_pitch = (uint32_t)p.slab * 4 + 16;
    const int prow = 1 << p.prow_log2;
    const uint32_t a_all = (uint32_t)p.nbuf * a_bytes;
    const uint32_t park0 = p.alias ? a_tile0 : a_tile0 + a_all;
    const uint32_t park = park0 + (uint32_t)(warp * prow) * park_pitch;
    const uint32_t table_off = p.alias ? max(a_all, p.park_bytes) : a_all + p.park_bytes;
    int32_t *s_cum = reinterpret_cast<int32_t *>(smem_raw + (a_tile0 - smem_u32(smem_raw)) + table_off);

    if (tid == 0) {
        mbar_init(bar, 1);
        fence_mbar_init();
    }
    if (warp == 0) tmem_alloc(smem_u32(&s_tmem), p.ncols);
    build_chunk_table(p.seg, p.K, s_cum, s_warp_sums);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = s_tmem;

    const int total = s_cum[p.K];
    const int per = (total + gridDim.x - 1) / gridDim.x;
    const int lo = blockIdx.x * per, hi = min(total, lo + per);
    // forward: B = W[tap] read MN-major (its rows are the contraction index c);
    // input gradient: B = W[tap] read K-major (its rows are the output index c)
    const uint32_t idesc = instr_desc(p.fmt, 128, outw, 0, p.transpose ? 0 : 1);
    const int ksteps = inw >> 4;
    uint32_t phase = 0;
    int loaded_tap = -1;
    bool alive = true;

    auto load_weight = [&](int tap) {
        const uint16_t *w = p.weight + (int64_t)tap * p.C * p.M;
        const int cpr = p.M >> 3;
        for (int e = tid; e < p.C * cpr; e += 128) {
            int c = e / cpr, ch = e - c * cpr;
            uint32_t dst = b_tile + (uint32_t)(ch >> 3) * w_blk + (uint32_t)c * 128 + (uint32_t)(((ch & 7) ^ (c & 7)) << 4);
            cp_async16(dst, w + (int64_t)c * p.M + ch * 8);
        }
    };

    ChunkCursor c0, c1, c2;  // chunk, chunk + 1, chunk + 2
    int pre_g = 0, pre_s = 0;
    if (lo < hi) {
        c0.seek(s_cum, p.seg, p.K, lo);
        c1 = c0;
        c2 = c0;
        const int rows = c0.rows(lo);
        if (tid < rows) {
            s_gather[0][tid] = p.gather[c0.first(lo) + tid];
            s_scatter[0][tid] = p.scatter[c0.first(lo) + tid];
        }
        load_weight(c0.tap);
        loaded_tap = c0.tap;
        __syncthreads();
        gather_tile<false>(a_tile0, p.feat, s_gather[0], rows, inw, tid, 128);
        cp_async_commit();
        if (lo + 1 < hi) {
            c1.advance(s_cum, p.seg, p.K, lo + 1);
            c2 = c1;
            if (tid < c1.rows(lo + 1)) {
                pre_g = p.gather[c1.first(lo + 1) + tid];
                pre_s = p.scatter[c1.first(lo + 1) + tid];
            }
        }
    }

    for (int chunk = lo; chunk < hi && alive; ++chunk) {
        const int b = (chunk - lo) & 1;
        const int rows = c0.rows(chunk);
        const bool have_next = chunk + 1 < hi;
        const int rows_next = have_next ? c1.rows(chunk + 1) : 0;
        if (have_next && tid < rows_next) {
            s_gather[b ^ 1][tid] = pre_g;
            s_scatter[b ^ 1][tid] = pre_s;
        }
        __syncthreads();
        if (have_next && two)
            gather_tile<false>(a_tile0 + (uint32_t)(b ^ 1) * a_bytes, p.feat, s_gather[b ^ 1], rows_next, inw, tid, 128);
        cp_async_commit();
        if (chunk + 2 < hi) {
            c2.advance(s_cum, p.seg, p.K, chunk + 2);
            if (tid < c2.rows(chunk + 2)) {
                pre_g = p.gather[c2.first(chunk + 2) + tid];
                pre_s = p.scatter[c2.first(chunk + 2) + tid];
            }
        }
        if (two) cp_async_wait<1>();  // everything but the gather just issued has landed
        else cp_async_wait<0>();
        fence_async_smem();
        __syncthreads();

        if (tid == 0) {
            tc_fence_after();
            const uint32_t a_tile = a_tile0 + (two ? (uint32_t)b * a_bytes : 0u);
            for (int s = 0; s < ksteps; ++s) {
                uint64_t ad = smem_desc(a_tile + (uint32_t)(s >> 2) * BLK_BYTES + (uint32_t)(s & 3) * 32, 16, 1024);
                uint64_t bd = p.transpose
                                  ? smem_desc(b_tile + (uint32_t)(s >> 2) * w_blk + (uint32_t)(s & 3) * 32, 16, 1024)
                                  : smem_desc(b_tile + (uint32_t)s * 2048, w_blk, 1024);
                tc_mma(tmem, ad, bd, idesc, s > 0 ? 1u : 0u);
            }
            tc_commit(bar);
        }
        alive = __syncthreads_and(mbar_wait(bar, phase, 1u, &g_device_status));
        phase ^= 1u;
        tc_fence_after();
        // the weight tile is free now: fetch the next tap's if the next chunk needs it
        if (have_next && c1.tap != loaded_tap) {
            load_weight(c1.tap);
            loaded_tap = c1.tap;
            cp_async_commit();
        }
        if (have_next && !two && !p.alias) {  // single A tile: it is free as well
            gather_tile<false>(a_tile0, p.feat, s_gather[b ^ 1], rows_next, inw, tid, 128);
            cp_async_commit();
        }
        if (BULK && alive && warp * 32 < rows) {
            const int row = warp * 32 + lane;
            const bool row_ok = row < rows;
            float *dst_row = p.acc + (int64_t)(row_ok ? s_scatter[b][row] : 0) * outw;
            // a warp parks `prow` rows at a time (32, or 16 when shared memory is better spent
            // on one more resident CTA): lanes of the current batch store, the others only
            // take part in the warp-wide TMEM load
            const uint32_t my_park = park + (uint32_t)(lane & (prow - 1)) * park_pitch;
            for (int batch = 0; batch * prow < 32; ++batch) {
                const bool mine = (lane >> p.prow_log2) == batch;
                if (warp * 32 + batch * prow >= rows) break;
                for (int col0 = 0; col0 < outw; col0 += p.slab) {
                    bulk_wait_read();  // the previous reductions have read this warp's parking area
                    __syncwarp();
                    for (int c32 = 0; c32 < p.slab; c32 += 32) {
                        float v[32];
                        tmem_ld32(tmem + ((uint32_t)(warp * 32) << 16) + (uint32_t)(col0 + c32), v);
                        if (mine) {
#pragma unroll
                            for (int q = 0; q < 8; ++q)
                                asm volatile("st.shared.v4.f32 [%0], {%1,%2,%3,%4};" ::"r"(my_park + (uint32_t)(c32 + 4 * q) * 4),
                                             "f"(v[4 * q]), "f"(v[4 * q + 1]), "f"(v[4 * q + 2]), "f"(v[4 * q + 3]) : "memory");
                        }
                    }
                    fence_async_smem();
                    const int cols = min(p.slab, outw - col0);
                    if (row_ok && mine) bulk_reduce_add_f32(dst_row + col0, my_park, (uint32_t)cols * 4);
                    bulk_commit();
                }
            }
        } else if (MODE == 2 && alive && warp * 32 < rows) {
            // one thread per accumulator row: 32 columns at a time, rounded and stored
            const int row = warp * 32 + lane;
            const bool row_ok = row < rows;
            uint16_t *dst_row = p.out + (int64_t)(row_ok ? s_scatter[b][row] : 0) * outw;
            for (int col0 = 0; col0 < outw; col0 += 32) {
                float v[32];
                tmem_ld32(tmem + ((uint32_t)(warp * 32) << 16) + (uint32_t)col0, v);
                if (row_ok) {
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        if (col0 + 8 * q < outw) {
                            uint4 o;
                            o.x = pack_pair(v[8 * q], v[8 * q + 1], p.fmt), o.y = pack_pair(v[8 * q + 2], v[8 * q + 3], p.fmt);
                            o.z = pack_pair(v[8 * q + 4], v[8 * q + 5], p.fmt), o.w = pack_pair(v[8 * q + 6], v[8 * q + 7], p.fmt);
                            *reinterpret_cast<uint4 *>(dst_row + col0 + 8 * q) = o;
                        }
                    }
                }
            }
        } else if (MODE == 0 && alive && warp * 32 < rows) {
            // wide rows: scatter from registers (two-float vector reductions); with several
            // 64-column blocks per row the single parking area would serialise the bulk reductions
            const int32_t *sc = s_scatter[b];
#pragma unroll 1
            for (int half = 0; half < 2; ++half) {
                if (warp * 32 + half * 16 >= rows) break;
                const int ra = warp * 32 + half * 16 + (lane >> 2), rb = ra + 8;
                const int64_t da = ra < rows ? sc[ra] : -1, db = rb < rows ? sc[rb] : -1;
                for (int col0 = 0; col0 < outw; col0 += 64) {
                    float v[32];
                    tmem_ld_16x64(tmem + ((uint32_t)(warp * 32 + half * 16) << 16) + (uint32_t)col0, v);
                    scatter_block(p.acc, da, db, outw, col0, lane, v);
                }
            }
        }
        if (p.alias) {
            // the parking area lies in the feature tile: gather the next chunk only after the
            // reductions have read it (other resident CTAs cover the latency)
            bulk_wait_read();
            __syncthreads();
            if (have_next) {
                gather_tile<false>(a_tile0, p.feat, s_gather[b ^ 1], rows_next, inw, tid, 128);
                cp_async_commit();
            }
        }
        c0 = c1;
        c1 = c2;
        tc_fence_before();
        __syncthreads();
    }
    cp_async_wait<0>();
    bulk_wait_read();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, p.ncols);
}

struct VvorTcParams {
    const uint16_t *a, *b;  // (n_a, Ma), (n_b, Cb)
    const int32_t *a_idx, *b_idx;
    const int64_t *seg;
    float *acc;             // (n_o, Ma, Cb)
    int n_o, Ma, Cb, fmt, stages;
    uint32_t ncols;
};

constexpr int MAX_STAGES = 4;

// Chunks of CHR triplets (the contraction length of one group of MMAs) through a ring of
// `stages` operand buffers.  NT threads.
//  * one stage, 128 threads: gather, multiply, gather ...; several CTAs per SM overlap each
//    other (narrow operands, where three and more CTAs fit).
//  * wide operands leave room for one or two CTAs per SM: more warps issue the copies of a
//    chunk, and with two or more stages the multiply of chunk n is issued BEFORE the CTA waits
//    for the multiply of chunk n-1 and refills its buffer, so the tensor core always has the
//    next group queued and the copies of the following chunks are in flight meanwhile.
template <int NT, int CHR, bool RING>
__global__ void __launch_bounds__(NT) vvor_tc_kernel(VvorTcParams p) {
    constexpr uint32_t BLK = CHR * 128;   // one 64-channel block of a CHR-row tile
    using Cursor = ChunkCursorT<CHR>;
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t s_bar[2];
    __shared__ uint32_t s_tmem;
    __shared__ int32_t s_warp_sums[NT / 32];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const int row_tiles = (p.Ma + 127) >> 7;
    const int ablk = (p.Ma + 63) >> 6;  // blocks actually filled; an odd count borrows the next block as padding
    const int bblk = (p.Cb + 63) >> 6;
    const uint32_t buf_bytes = (uint32_t)(ablk + bblk) * BLK;
    const int NS = RING ? p.stages : 1;   // RING: two to four stages
    // behind the operand stages: the index rings of both operands, then the chunk table
    // (the ring keeps the index rows of 2 NS chunks: they are fetched NS-1 iterations before the copies that use them)
    const int IR = RING ? 2 * NS : 1;
    int32_t(*s_ia)[CHR] = reinterpret_cast<int32_t(*)[CHR]>(smem_raw + (base - smem_u32(smem_raw)) + (size_t)NS * buf_bytes);
    int32_t(*s_ib)[CHR] = s_ia + IR;
    int32_t *s_cum = reinterpret_cast<int32_t *>(s_ib + IR);
    const uint32_t bar0 = smem_u32(&s_bar[0]), bar1 = smem_u32(&s_bar[1]);

    if (tid == 0) {
        mbar_init(bar0, 1);
        mbar_init(bar1, 1);
        fence_mbar_init();
    }
    if (warp == 0) tmem_alloc(smem_u32(&s_tmem), p.ncols);
    build_chunk_table<CHR>(p.seg, p.n_o, s_cum, s_warp_sums);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = s_tmem;

    const int total = s_cum[p.n_o];
    const int per = (total + gridDim.x - 1) / gridDim.x;
    const int lo = blockIdx.x * per, hi = min(total, lo + per);
    const uint32_t idesc = instr_desc(p.fmt, 128, p.Cb, 1, 1);
    bool alive = true;
    bool fresh = true;  // next MMA starts a new accumulation

    Cursor cur, pre;  // chunk being multiplied; chunk whose indices are being fetched
    int pre_a = 0, pre_b = 0;
    auto stage_indices = [&](const Cursor &cc, int chunk, int slot, bool from_regs) {
        const int rows = cc.rows(chunk);
        if (tid < rows) {
            s_ia[slot][tid] = from_regs ? pre_a : p.a_idx[cc.first(chunk) + tid];
            s_ib[slot][tid] = from_regs ? pre_b : p.b_idx[cc.first(chunk) + tid];
        }
        return rows;
    };
    auto copy_rows = [&](int slot, int rows) {
        __syncthreads();
        const uint32_t a_tile = base + (uint32_t)slot * buf_bytes;
        gather_tile<true, CHR>(a_tile, p.a, s_ia[slot], rows, p.Ma, tid, NT);
        gather_tile<true, CHR>(a_tile + (uint32_t)ablk * BLK, p.b, s_ib[slot], rows, p.Cb, tid, NT);
    };
    auto issue_gather = [&](const Cursor &cc, int chunk, int slot, bool from_regs) {
        copy_rows(slot, stage_indices(cc, chunk, slot, from_regs));
    };
    auto prefetch_indices = [&](int chunk) {
        if (chunk < hi) {
            pre.advance(s_cum, p.seg, p.n_o, chunk);
            if (tid < pre.rows(chunk)) {
                pre_a = p.a_idx[pre.first(chunk) + tid];
                pre_b = p.b_idx[pre.first(chunk) + tid];
            }
        }
    };
    auto wait_landed = [&]() {  // the oldest chunk in the ring has landed once NS-1 newer groups are pending
        if (NS == 1) cp_async_wait<0>();
        else if (NS == 2) cp_async_wait<1>();
        else if (NS == 3) cp_async_wait<2>();
        else cp_async_wait<3>();
        fence_async_smem();
        __syncthreads();
    };
    auto multiply = [&](int slot, int rows, uint32_t bar) {  // one thread
        tc_fence_after();
        const uint32_t a_tile = base + (uint32_t)slot * buf_bytes;
        const uint32_t b_tile = a_tile + (uint32_t)ablk * BLK;
        const int ksteps = (rows + 15) >> 4;
        for (int rt = 0; rt < row_tiles; ++rt) {
            for (int s = 0; s < ksteps; ++s) {
                uint64_t ad = smem_desc(a_tile + (uint32_t)(rt * 2) * BLK + (uint32_t)s * 2048, BLK, 1024);
                uint64_t bd = smem_desc(b_tile + (uint32_t)s * 2048, BLK, 1024);
                tc_mma(tmem + (uint32_t)(rt * p.Cb), ad, bd, idesc, (fresh && s == 0) ? 0u : 1u);
            }
        }
        tc_commit(bar);
    };
    // a warp reads the 32 TMEM lanes of its quarter (warp % 4); the warps of a quarter share its columns
    const int quarter = warp & 3, col_part = warp >> 2;
    auto flush_tap = [&](int o) {
        float *dst_o = p.acc + (int64_t)o * p.Ma * p.Cb;
        for (int rt = 0; rt < row_tiles; ++rt) {
#pragma unroll 1
            for (int half = 0; half < 2; ++half) {
                const int m0 = rt * 128 + quarter * 32 + half * 16;
                if (m0 >= p.Ma) break;
                const int ma = m0 + (lane >> 2), mb = ma + 8;
                const int64_t da = ma < p.Ma ? ma : -1, db = mb < p.Ma ? mb : -1;
                for (int c0 = col_part * 64; c0 < p.Cb; c0 += (NT / 128) * 64) {
                    float v[32];
                    tmem_ld_16x64(tmem + ((uint32_t)(quarter * 32 + half * 16) << 16) + (uint32_t)(rt * p.Cb + c0), v);
                    scatter_block(dst_o, da, db, p.Cb, c0, lane, v);
                }
            }
        }
    };
    int pending_tap = -1;  // tap whose last MMA has been issued but whose sums are still in TMEM

    if (!RING) {
        uint32_t phase = 0;
        if (lo < hi) {
            cur.seek(s_cum, p.seg, p.n_o, lo);
            pre = cur;
            prefetch_indices(lo);
        }
        for (int chunk = lo; chunk < hi && alive; ++chunk) {
            // the MMA of the previous chunk must be done before the buffer is refilled
            if (chunk > lo) {
                alive = __syncthreads_and(mbar_wait(bar0, phase, 2u, &g_device_status));
                phase ^= 1u;
                tc_fence_after();
                if (alive && pending_tap >= 0) {
                    flush_tap(pending_tap);
                    pending_tap = -1;
                    fresh = true;
                    tc_fence_before();
                }
            }
            issue_gather(pre, chunk, 0, true);
            cp_async_commit();
            prefetch_indices(chunk + 1);
            wait_landed();
            cur.advance(s_cum, p.seg, p.n_o, chunk);
            if (tid == 0 && alive) multiply(0, cur.rows(chunk), bar0);
            fresh = false;
            if ((chunk + 1 == hi) || cur.last_of_tap(chunk)) pending_tap = cur.tap;
        }
        if (lo < hi && alive) {
            alive = __syncthreads_and(mbar_wait(bar0, phase, 2u, &g_device_status));
            tc_fence_after();
            if (alive && pending_tap >= 0) flush_tap(pending_tap);
        }
    } else {
        // Warp 0 issues the multiplies; warps 1 .. NT/32-1 copy.  One block barrier per iteration
        // (the copies of all threads must be visible before the multiply reads the stage); the
        // completion of a multiply is observed by every thread on the mbarrier itself.
        constexpr int NCOPY = NT - 32;
        const int ctid = tid - 32;           // copy thread number (negative: warp 0)
        uint32_t phase0 = 0u, phase1 = 0u;   // parities of the two barriers (multiplies of even / odd chunks)
        auto wait_multiply_all = [&](int n) {    // with a block barrier: every thread knows the outcome
            const bool odd = n & 1;
            const bool ok = __syncthreads_and(mbar_wait(odd ? bar1 : bar0, odd ? phase1 : phase0, 2u, &g_device_status));
            if (odd) phase1 ^= 1u; else phase0 ^= 1u;
            return ok;
        };
        auto wait_multiply_self = [&](int n) {   // this thread only
            const bool odd = n & 1;
            const bool ok = mbar_wait(odd ? bar1 : bar0, odd ? phase1 : phase0, 2u, &g_device_status);
            if (odd) phase1 ^= 1u; else phase0 ^= 1u;
            return ok;
        };
        // Index rows of chunk `chunk` into slot `islot` of the index ring, as 4-byte asynchronous
        // copies in the caller's copy group: a plain load would come back behind the tens of KB of
        // row copies already queued in the SM's memory pipeline.
        auto fetch_indices = [&](int chunk, int islot) {
            if (chunk < hi) {
                pre.advance(s_cum, p.seg, p.n_o, chunk);
                if (ctid >= 0 && ctid < pre.rows(chunk)) {
                    const int64_t t = pre.first(chunk) + ctid;
                    cp_async4(smem_u32(&s_ia[islot][ctid]), p.a_idx + t);
                    cp_async4(smem_u32(&s_ib[islot][ctid]), p.b_idx + t);
                }
            }
        };
        Cursor fill;   // chunk whose rows are being copied
        auto copy_chunk = [&](int chunk, int slot, int islot) {   // its index rows have landed
            fill.advance(s_cum, p.seg, p.n_o, chunk);
            const int rows = fill.rows(chunk);
            if (ctid >= 0) {
                const uint32_t a_tile = base + (uint32_t)slot * buf_bytes;
                gather_tile<true, CHR>(a_tile, p.a, s_ia[islot], rows, p.Ma, ctid, NCOPY);
                gather_tile<true, CHR>(a_tile + (uint32_t)ablk * BLK, p.b, s_ib[islot], rows, p.Cb, ctid, NCOPY);
            }
        };
        auto next = [](int v, int mod) { return v + 1 == mod ? 0 : v + 1; };
        int st_mma = 0, st_fill = NS - 1, ix_fill = NS - 1, ix_fetch = 2 * (NS - 1);   // all < IR = 2 NS
        if (lo < hi) {
            cur.seek(s_cum, p.seg, p.n_o, lo);
            pre = cur;
            fill = cur;
            // prologue: index rows of chunks 0 .. 2(NS-1)-1, then the rows of chunks 0 .. NS-2
            for (int m = 0; m < 2 * (NS - 1); ++m) fetch_indices(lo + m, m);
            cp_async_commit();
            cp_async_wait<0>();
            __syncthreads();
            for (int m = 0; m < NS - 1; ++m) {
                if (lo + m < hi) copy_chunk(lo + m, m, m);
                cp_async_commit();
            }
        }
        // Iteration n: [flush a closed tap] - chunk n landed - multiply n - multiply n-1 done? -
        // refill its stage with chunk n+NS-1 and fetch the index rows of chunk n+2(NS-1).  NS-1 copy
        // groups before the loop and one per iteration, committed after the iteration's wait: chunk
        // n (and the index rows fetched NS-1 iterations ago, which this iteration's copies read)
        // has landed once at most NS-2 groups are pending.
        bool failed = false;   // this thread's wait ran out; the block leaves the loop together at the barrier
        for (int chunk = lo; chunk < hi; ++chunk) {
            const int n = chunk - lo;
            bool prev_waited = n == 0;
            if (n > 0 && pending_tap >= 0) {
                // the previous chunk closed its tap: its sums leave TMEM before this chunk starts a new one
                alive = wait_multiply_all(n - 1);
                prev_waited = true;
                if (!alive) break;
                tc_fence_after();
                flush_tap(pending_tap);
                pending_tap = -1;
                fresh = true;
                tc_fence_before();
            }
            if (NS == 2) cp_async_wait<0>();
            else if (NS == 3) cp_async_wait<1>();
            else cp_async_wait<2>();
            fence_async_smem();
            if (__syncthreads_or(failed)) {
                alive = false;
                break;
            }
            cur.advance(s_cum, p.seg, p.n_o, chunk);
            if (tid == 0) multiply(st_mma, cur.rows(chunk), (n & 1) ? bar1 : bar0);
            fresh = false;
            if (!prev_waited) failed = !wait_multiply_self(n - 1);
            // the stage of chunk n-1 (for n = 0: the one the prologue left empty) is free
            if (!failed) {
                if (chunk + NS - 1 < hi) copy_chunk(chunk + NS - 1, st_fill, ix_fill);
                fetch_indices(chunk + 2 * (NS - 1), ix_fetch);
            }
            cp_async_commit();
            st_mma = next(st_mma, NS), st_fill = next(st_fill, NS);
            ix_fill = next(ix_fill, IR), ix_fetch = next(ix_fetch, IR);
            if ((chunk + 1 == hi) || cur.last_of_tap(chunk)) pending_tap = cur.tap;
        }
        if (lo < hi && alive) {
            alive = wait_multiply_all(hi - 1 - lo) && !__syncthreads_or(failed);
            tc_fence_after();
            if (alive && pending_tap >= 0) flush_tap(pending_tap);
        }
    }
    cp_async_wait<0>();
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, p.ncols);
}

uint32_t pow2_cols(int n) {
    uint32_t c = 32;
    while ((int)c < n) c <<= 1;
    return c;
}

// CTAs per SM: bounded by shared memory (227 KiB usable, 1 KiB reserved per
// CTA), by TMEM (512 columns) and by registers / warp slots.
int ctas_per_sm(size_t smem, uint32_t ncols, int regs_per_thread, int threads = 128) {
    int by_smem = (int)((size_t)232448 / (smem + 1024));
    int by_tmem = (int)(512 / ncols);
    int by_regs = 65536 / (((regs_per_thread * 32 + 255) / 256 * 256) * (threads / 32));
    int occ = std::min(by_smem, std::min(by_tmem, by_regs));
    if (occ > 8) occ = 8;
    return occ < 1 ? 1 : occ;
}

// Registers per thread of a kernel (asked once per kernel; the persistent grids
// must not exceed what is resident at once, or the surplus CTAs run as a second wave).
template <typename Kernel>
int kernel_registers(Kernel kernel, int *cached) {
    if (*cached == 0) {
        cudaFuncAttributes attr;
        *cached = cudaFuncGetAttributes(&attr, kernel) == cudaSuccess ? attr.numRegs : 128;
    }
    return *cached;
}

// Dynamic shared memory padded so that at most 512 / ncols CTAs share an SM
// (their TMEM allocations then always fit).
size_t pad_for_tmem(size_t smem, uint32_t ncols) {
    size_t max_ctas = 512 / ncols;
    size_t floor_bytes = (size_t)232448 / (max_ctas + 1) + 1024;
    return smem > floor_bytes ? smem : floor_bytes;
}

// cudaFuncSetAttribute is a host-side round trip; raise the opt-in shared-memory
// limit of a kernel only when a launch needs more than any launch before it.
template <typename Kernel>
int ensure_dynamic_smem(Kernel kernel, size_t smem, int *granted) {
    if ((int)smem <= *granted) return PCX_OK;
    PCX_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    PCX_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
    *granted = (int)smem;
    return PCX_OK;
}

bool aligned16(const void *p) { return ((uintptr_t)p & 15) == 0; }

}  // namespace

bool mvmr_tensor_supported(const MvmrArgs &a) {
    if (a.dtype != PCX_F16 && a.dtype != PCX_BF16) return false;
    if (a.G != 1 || !a.seg_offs || a.T <= 0 || a.K > MAX_TAPS_SMEM) return false;
    const int inw = a.transpose ? a.M : a.C, outw = a.transpose ? a.C : a.M;
    if (inw % 16 || outw % 16 || inw < 16 || outw < 16 || inw > 256 || outw > 256) return false;
    if (!aligned16(a.weight) || !aligned16(a.feat)) return false;
    if (a.T / CH + a.K >= INT32_MAX) return false;
    return true;
}

bool vvor_tensor_supported(const VvorArgs &a) {
    if (a.dtype != PCX_F16 && a.dtype != PCX_BF16) return false;
    if (a.G != 1 || !a.seg_offs || a.T <= 0 || a.n_o > MAX_TAPS_SMEM) return false;
    if (a.Ma % 16 || a.Cb % 16 || a.Ma < 16 || a.Cb < 16 || a.Ma > 256 || a.Cb > 256) return false;
    if (((a.Ma + 127) / 128 - 1) * a.Cb + (a.Cb + 63) / 64 * 64 > 512) return false;
    if (!aligned16(a.a) || !aligned16(a.b)) return false;
    return true;
}

int mvmr_tensor(const MvmrArgs &a, cudaStream_t stream) {
    const int inw = a.transpose ? a.M : a.C, outw = a.transpose ? a.C : a.M;
    MvmrTcParams p;
    p.weight = (const uint16_t *)a.weight, p.feat = (const uint16_t *)a.feat;
    p.gather = a.gather, p.scatter = a.scatter, p.seg = a.seg_offs, p.acc = a.acc;
    p.out = (uint16_t *)a.out_rows;
    p.K = a.K, p.C = a.C, p.M = a.M, p.transpose = a.transpose, p.fmt = a.dtype == PCX_BF16 ? 1 : 0;
    p.ncols = pow2_cols((outw + 63) / 64 * 64);  // the epilogue reads blocks of up to 64 columns
    // Measured on B200: rows of exactly 64 floats leave fastest through one bulk reduction
    // each (64 vs 84 us on the 150k-point scene); narrower and wider rows from registers
    // (C = 32: 50 vs 59 us, C = 128: 160 vs 180 us, C = 256: 390 vs 671 us).  Folding rows
    // with equal destinations in shared memory first was tried and cost more than it saved.
    bool bulk = outw == 64;
    if (const char *e = getenv("PCX_MVMR_SCATTER")) bulk = atoi(e) != 0;
    const bool store = a.out_rows != nullptr;
    if (store) bulk = false;
    const int kb = (inw + 63) / 64, wb = (a.M + 63) / 64;
    const size_t static_smem = 2176;  // index rings, barrier
    const size_t table = align_up((size_t)(a.K + 1) * 4, 16);
    p.slab = outw >= 64 ? 64 : 32;  // columns parked per bulk reduction
    // Rows a warp parks at a time.  Fewer rows leave shared memory for more resident CTAs,
    // which hide the gather latency (measured on the 150k-point scene, C = 64: 32 rows /
    // 3 CTAs per SM 78 us, 16 rows / 5 CTAs 64 us, 8 rows / 6 CTAs 66 us).
    p.prow_log2 = 4;
    if (const char *e = getenv("PCX_MVMR_PARK_ROWS")) p.prow_log2 = atoi(e) == 32 ? 5 : atoi(e) == 8 ? 3 : 4;
    p.park_bytes = bulk ? (uint32_t)(4 << p.prow_log2) * (p.slab * 4 + 16) : 0;
    // The parking area shares the feature tile's memory: the next gather then waits for the
    // reductions to drain, but one more CTA fits per SM (measured: 62 vs 65 us).
    p.alias = bulk ? 1 : 0;
    if (const char *e = getenv("PCX_MVMR_ALIAS")) p.alias = bulk && atoi(e) != 0;
    const size_t rest = 1024 + (size_t)wb * a.C * 128 + (p.alias ? 0 : p.park_bytes) + table;
    // One A tile: it is free again as soon as the multiply has finished, so the
    // next gather still overlaps the scatter, and more CTAs fit on an SM.
    p.nbuf = 1;
    if (const char *e = getenv("PCX_MVMR_NBUF"))
        if (atoi(e) == 2 && rest + 2 * (size_t)kb * BLK_BYTES + static_smem <= 232448 - 1024) p.nbuf = 2;
    if (p.alias) p.nbuf = 1;
    size_t smem = rest + std::max((size_t)p.nbuf * kb * BLK_BYTES, p.alias ? (size_t)p.park_bytes : (size_t)0);
    smem = pad_for_tmem(smem, p.ncols);
    if (smem + static_smem > 232448 - 1024) PCX_FAIL(PCX_E_UNSUPPORTED, "mvmr tensor kernel does not fit (smem %zu)", smem);
    static int granted_mvmr[3][64] = {};   // per output mode and device
    int dev = 0;
    PCX_CUDA(cudaGetDevice(&dev));
    if (int rc = store ? ensure_dynamic_smem(mvmr_tc_kernel<2>, smem, &granted_mvmr[2][dev & 63])
                 : bulk ? ensure_dynamic_smem(mvmr_tc_kernel<1>, smem, &granted_mvmr[1][dev & 63])
                        : ensure_dynamic_smem(mvmr_tc_kernel<0>, smem, &granted_mvmr[0][dev & 63]))
        return rc;
    static int regs_mvmr[3] = {0, 0, 0};
    const int regs = store ? kernel_registers(mvmr_tc_kernel<2>, &regs_mvmr[2])
                     : bulk ? kernel_registers(mvmr_tc_kernel<1>, &regs_mvmr[1])
                            : kernel_registers(mvmr_tc_kernel<0>, &regs_mvmr[0]);
    const int occ = ctas_per_sm(smem + static_smem, p.ncols, regs);
    int64_t upper = a.T / CH + a.K + 1;
    int64_t grid = std::min<int64_t>(upper, (int64_t)occ * num_sms());
    prof_begin(store ? (a.transpose ? "mvmr_tc_kernel(dgrad, store)" : "mvmr_tc_kernel(fwd, store)")
                     : (a.transpose ? "mvmr_tc_kernel(dgrad)" : "mvmr_tc_kernel(fwd)"), stream);
    if (store) mvmr_tc_kernel<2><<<(unsigned)grid, 128, smem, stream>>>(p);
    else if (bulk) mvmr_tc_kernel<1><<<(unsigned)grid, 128, smem, stream>>>(p);
    else mvmr_tc_kernel<0><<<(unsigned)grid, 128, smem, stream>>>(p);
    prof_end(stream);
    PCX_LAUNCH_CHECK();
    return PCX_OK;
}

// One instantiation of the VVOR kernel: its shared-memory opt-in, its resident CTAs, its launch.
template <int NT, int CHR, bool RING>
int launch_vvor(const VvorTcParams &p, int64_t chunks_upper, size_t smem, size_t static_smem, cudaStream_t stream) {
    static int granted[64] = {};   // per device
    static int regs = 0;
    int dev = 0;
    PCX_CUDA(cudaGetDevice(&dev));
    if (int rc = ensure_dynamic_smem(vvor_tc_kernel<NT, CHR, RING>, smem, &granted[dev & 63])) return rc;
    const int occ = ctas_per_sm(smem + static_smem, p.ncols, kernel_registers(vvor_tc_kernel<NT, CHR, RING>, &regs), NT);
    const int64_t grid = std::min<int64_t>(chunks_upper, (int64_t)occ * num_sms());
    prof_begin("vvor_tc_kernel", stream);
    vvor_tc_kernel<NT, CHR, RING><<<(unsigned)grid, NT, smem, stream>>>(p);
    prof_end(stream);
    PCX_LAUNCH_CHECK();
    return PCX_OK;
}

int vvor_tensor(const VvorArgs &a, cudaStream_t stream) {
    VvorTcParams p;
    p.a = (const uint16_t *)a.a, p.b = (const uint16_t *)a.b, p.a_idx = a.a_idx, p.b_idx = a.b_idx;
    p.seg = a.seg_offs, p.acc = a.acc;
    p.n_o = (int)a.n_o, p.Ma = a.Ma, p.Cb = a.Cb, p.fmt = a.dtype == PCX_BF16 ? 1 : 0;
    const int row_tiles = (a.Ma + 127) / 128;
    p.ncols = pow2_cols((row_tiles - 1) * a.Cb + (a.Cb + 63) / 64 * 64);  // flushed in blocks of 64 columns
    const size_t blocks = (size_t)((a.Ma + 63) / 64 + (a.Cb + 63) / 64);
    // one stage = both operand tiles plus their index rows
    // (index rows: two per stage and operand, the ring variant fetches them ahead of the copies)
    auto stage_bytes = [&](int chr) { return blocks * (size_t)chr * 128 + 4 * (size_t)chr * sizeof(int32_t); };
    const size_t fixed = 1024 + align_up((size_t)(a.n_o + 1) * 4, 16);  // alignment slack, chunk table
    const size_t static_smem = 160;  // barriers, TMEM address, scan scratch
    // Measured on B200 (27 taps, 3.2 M triplets over 90 000 rows; ms per call):
    //  * three and more CTAs fit on an SM (narrow operands): chunks of 128 triplets, one stage, 128
    //    threads -- more resident CTAs hide the gather latency better than a ring inside fewer CTAs;
    //  * two fit (192 x 128, 256 x 128, 192 x 96): the same with 256 threads, 0.37 / 0.36 / 0.39
    //    (ring of 64-triplet chunks in two CTAs 0.43 / 0.39 / 0.45, in one CTA of 512 threads 0.52 / 0.48 / 0.56);
    //  * one fits (256 x 256: all of tensor memory): chunks of 64 triplets through a ring as deep
    //    as fits (3 stages), 512 threads, 0.52 (one stage of 128 triplets: 0.63 with 512 threads,
    //    0.83 with 128).
    const int by_memory = ctas_per_sm(fixed + stage_bytes(128) + static_smem, p.ncols, 32);
    int chr = by_memory >= 2 ? 128 : 64;
    int threads = by_memory >= 3 ? 128 : by_memory == 2 ? 256 : 512;
    if (const char *e = getenv("PCX_VVOR_CHUNK")) {
        const int want = atoi(e);
        if (want == 64 || want == 128) chr = want;
    }
    if (const char *e = getenv("PCX_VVOR_THREADS")) {
        const int want = atoi(e);
        if (want == 128 || want == 256 || want == 512) threads = want;
    }
    const size_t budget = by_memory >= 2 && threads <= 256 ? 232448 / 2 : 232448;   // keep two CTAs per SM where two fit
    int max_fit = 1;
    for (int ns = chr == 128 ? 1 : MAX_STAGES; ns >= 1; --ns)
        if (fixed + ns * stage_bytes(chr) + static_smem + 1024 <= budget) {
            max_fit = ns;
            break;
        }
    int stages = chr == 128 ? 1 : max_fit;
    if (const char *e = getenv("PCX_VVOR_STAGES")) {
        const int want = atoi(e);
        if (want >= 1 && want <= max_fit) stages = want;
    }
    p.stages = stages;
    size_t smem = fixed + stages * stage_bytes(chr);
    smem = pad_for_tmem(smem, p.ncols);
    if (smem + static_smem > 232448 - 1024) PCX_FAIL(PCX_E_UNSUPPORTED, "vvor tensor kernel does not fit (smem %zu)", smem);
    const int64_t upper = a.T / chr + a.n_o + 1;
    if (chr == 128) {
        if (threads == 128) return launch_vvor<128, 128, false>(p, upper, smem, static_smem, stream);
        if (threads == 256) return launch_vvor<256, 128, false>(p, upper, smem, static_smem, stream);
        return launch_vvor<512, 128, false>(p, upper, smem, static_smem, stream);
    }
    if (stages == 1) {
        if (threads == 128) return launch_vvor<128, 64, false>(p, upper, smem, static_smem, stream);
        if (threads == 256) return launch_vvor<256, 64, false>(p, upper, smem, static_smem, stream);
        return launch_vvor<512, 64, false>(p, upper, smem, static_smem, stream);
    }
    if (threads <= 256) return launch_vvor<256, 64, true>(p, upper, smem, static_smem, stream);   // the ring wants the warps
    return launch_vvor<512, 64, true>(p, upper, smem, static_smem, stream);
}

// Device address of the status word, for kernels of other translation units.
int device_status_address(unsigned int **d_status) {
    PCX_CUDA(cudaGetSymbolAddress((void **)d_status, g_device_status));
    return PCX_OK;
}

int read_device_status(unsigned int *h_status, bool clear, cudaStream_t stream) {
    PCX_CUDA(cudaStreamSynchronize(stream));
    PCX_CUDA(cudaMemcpyFromSymbol(h_status, g_device_status, sizeof(unsigned int)));
    if (clear && *h_status) {
        unsigned int zero = 0;
        PCX_CUDA(cudaMemcpyToSymbol(g_device_status, &zero, sizeof(unsigned int)));
    }
    return PCX_OK;
}

}  // namespace pcx
