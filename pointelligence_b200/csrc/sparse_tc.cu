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
//   MVMR   D[128 triplets x N] = A[128 x Kc] * B[N x Kc]^T
//          A = gathered feature rows   (K-major: a row is contiguous along Kc)
//          B = weight tile of the tap  (K-major rows of the output channel)
//          epilogue: TMEM -> registers -> padded smem -> per-row run-merged
//          red.global.add.f32 (128 contiguous bytes per warp instruction).
//   VVOR   D[Ma x Cb] += X[t x Ma]^T * G[t x Cb], t = triplets of the chunk
//          both operands MN-major (a gathered row is contiguous along M / N,
//          the triplet index is the contraction), accumulated in TMEM over all
//          chunks of a tap and flushed once per (CTA, tap).
//
// One thread issues tcgen05.mma; completion is signalled with tcgen05.commit on
// an mbarrier.  Every wait is bounded: after the limit the kernel raises a flag
// in the status word, frees its TMEM and returns.
#include "sparse_kernels.cuh"

namespace pcx {

__device__ unsigned int g_device_status = 0;

namespace {

constexpr int CH = 128;            // triplets per chunk
constexpr int BLK_BYTES = CH * 128; // one 64-channel block of a 128-row tile
constexpr int STAGE_PITCH = 33;    // floats per row of the epilogue staging tile
constexpr uint32_t WAIT_LIMIT = 1u << 24;

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() {
    asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;" ::: "memory");
}
__device__ __forceinline__ void fence_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait; false (and the status flag) when the limit is hit.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, unsigned flag) {
    for (uint32_t it = 0; it < WAIT_LIMIT; ++it)
        if (mbar_try_wait(bar, parity)) return true;
    atomicOr(&g_device_status, flag);
    return false;
}
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_mma(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                       uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float *v) {
    uint32_t r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

// Shared-memory matrix descriptor, SWIZZLE_128B, descriptor version 1.
//   K-major operand : lbo = 1 (unused), sbo = bytes between 8-row groups
//   MN-major operand: lbo = bytes between 64-element blocks along M/N,
//                     sbo = bytes between groups of 8 contraction rows
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((addr >> 4) & 0x3fff);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3fff) << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3fff) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

// Instruction descriptor of tcgen05.mma.kind::f16 with fp32 accumulation.
__device__ __forceinline__ uint32_t instr_desc(int fmt /*0 f16, 1 bf16*/, int m, int n, int a_mn, int b_mn) {
    uint32_t d = 0;
    d |= 1u << 4;                       // D is fp32
    d |= (uint32_t)fmt << 7;            // A format
    d |= (uint32_t)fmt << 10;           // B format
    d |= (uint32_t)a_mn << 15;          // A major: 0 = K, 1 = MN
    d |= (uint32_t)b_mn << 16;          // B major
    d |= (uint32_t)(n >> 3) << 17;
    d |= (uint32_t)(m >> 4) << 24;
    return d;
}

// Position of a CTA in the chunk sequence; the bounds of the current tap are
// kept in registers and reloaded only when the chunk index leaves the tap.
struct ChunkCursor {
    int tap;
    int cum_lo, cum_hi;
    int64_t seg_lo, seg_hi;
    __device__ __forceinline__ void load(const int32_t *__restrict__ cum, const int64_t *__restrict__ seg) {
        cum_lo = cum[tap], cum_hi = cum[tap + 1];
        seg_lo = seg[tap], seg_hi = seg[tap + 1];
    }
    __device__ __forceinline__ void seek(const int32_t *__restrict__ cum, const int64_t *__restrict__ seg,
                                         int K, int chunk) {
        int lo = 0, hi = K;
        while (hi - lo > 1) {
            int mid = (lo + hi) >> 1;
            if (cum[mid] <= chunk) lo = mid; else hi = mid;
        }
        tap = lo;
        load(cum, seg);
    }
    __device__ __forceinline__ void advance(const int32_t *__restrict__ cum, const int64_t *__restrict__ seg,
                                            int K, int chunk) {
        if (chunk < cum_hi) return;
        while (tap + 1 < K && cum[tap + 1] <= chunk) ++tap;
        load(cum, seg);
    }
    __device__ __forceinline__ int64_t first(int chunk) const { return seg_lo + (int64_t)(chunk - cum_lo) * CH; }
    __device__ __forceinline__ int rows(int chunk) const {
        int64_t left = seg_hi - first(chunk);
        return (int)(left < CH ? left : CH);
    }
    __device__ __forceinline__ bool last_of_tap(int chunk) const { return chunk + 1 >= cum_hi; }
};

// Gather `rows` rows of `width` 2-byte channels into a swizzled tile; the row
// indices were staged in shared memory beforehand so that the copy loop issues
// cp.async back to back.  Rows past `rows` are zero-filled when ZERO_TAIL
// (needed when the row index is the contraction index), untouched otherwise.
template <bool ZERO_TAIL>
__device__ __forceinline__ void gather_tile(uint32_t tile, const uint16_t *__restrict__ src,
                                            const int32_t *s_idx, int rows, int width, int tid, int nthreads) {
    const int cpr = width >> 3;  // 16-byte pieces per row
    const int total = (ZERO_TAIL ? CH : rows) * cpr;
    for (int e = tid; e < total; e += nthreads) {
        int r = e / cpr, ch = e - r * cpr;
        uint32_t dst = tile + (uint32_t)(ch >> 3) * BLK_BYTES + (uint32_t)r * 128 + (uint32_t)(((ch & 7) ^ (r & 7)) << 4);
        if (r < rows) {
            cp_async16(dst, src + (int64_t)s_idx[r] * width + ch * 8);
        } else if (ZERO_TAIL) {
            asm volatile("st.shared.v4.b32 [%0], {%1,%1,%1,%1};" ::"r"(dst), "r"(0) : "memory");
        }
    }
}

struct MvmrTcParams {
    const uint16_t *bmat;   // (K, outw, inw) rows of output channel, contraction contiguous
    const uint16_t *feat;
    const int32_t *gather, *scatter;
    const int64_t *seg;
    const int32_t *cum;
    float *acc;
    int K, inw, outw, fmt;
    uint32_t ncols;
};

__global__ void __launch_bounds__(128) mvmr_tc_kernel(MvmrTcParams p) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t s_bar;
    __shared__ uint32_t s_tmem;
    __shared__ int32_t s_scatter[CH], s_gather[CH];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const int kb = (p.inw + 63) >> 6;
    const uint32_t a_tile = base;
    const uint32_t b_tile = a_tile + (uint32_t)kb * BLK_BYTES;
    const uint32_t b_blk = (uint32_t)p.outw * 128;
    float *stage = reinterpret_cast<float *>(smem_raw + (b_tile + (uint32_t)kb * b_blk - smem_u32(smem_raw)));
    const uint32_t bar = smem_u32(&s_bar);

    if (tid == 0) {
        mbar_init(bar, 1);
        fence_mbar_init();
    }
    if (warp == 0) tmem_alloc(smem_u32(&s_tmem), p.ncols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = s_tmem;

    const int total = p.cum[p.K];
    const int per = (total + gridDim.x - 1) / gridDim.x;
    const int lo = blockIdx.x * per, hi = min(total, lo + per);
    const uint32_t idesc = instr_desc(p.fmt, 128, p.outw, 0, 0);
    const int ksteps = p.inw >> 4;
    uint32_t phase = 0;
    int loaded_tap = -1;
    bool alive = true;
    ChunkCursor cur;
    if (lo < hi) cur.seek(p.cum, p.seg, p.K, lo);

    for (int chunk = lo; chunk < hi && alive; ++chunk) {
        cur.advance(p.cum, p.seg, p.K, chunk);
        const int tap = cur.tap;
        const int64_t t0 = cur.first(chunk);
        const int rows = cur.rows(chunk);
        if (tid < rows) {
            s_gather[tid] = p.gather[t0 + tid];
            s_scatter[tid] = p.scatter[t0 + tid];
        }

        if (tap != loaded_tap) {  // weight tile of this tap, rows = output channels
            const uint16_t *w = p.bmat + (int64_t)tap * p.outw * p.inw;
            const int cpr = p.inw >> 3;
            for (int e = tid; e < p.outw * cpr; e += 128) {
                int n = e / cpr, ch = e - n * cpr;
                uint32_t dst = b_tile + (uint32_t)(ch >> 3) * b_blk + (uint32_t)n * 128 + (uint32_t)(((ch & 7) ^ (n & 7)) << 4);
                cp_async16(dst, w + (int64_t)n * p.inw + ch * 8);
            }
            loaded_tap = tap;
        }
        __syncthreads();
        gather_tile<false>(a_tile, p.feat, s_gather, rows, p.inw, tid, 128);
        cp_async_wait_all();
        fence_async_smem();
        __syncthreads();

        if (tid == 0) {
            tc_fence_after();
            for (int s = 0; s < ksteps; ++s) {
                uint32_t off = (uint32_t)(s >> 2);
                uint64_t ad = smem_desc(a_tile + off * BLK_BYTES + (uint32_t)(s & 3) * 32, 16, 1024);
                uint64_t bd = smem_desc(b_tile + off * b_blk + (uint32_t)(s & 3) * 32, 16, 1024);
                tc_mma(tmem, ad, bd, idesc, s > 0 ? 1u : 0u);
            }
            tc_commit(bar);
        }
        alive = mbar_wait(bar, phase, 1u);
        phase ^= 1u;
        tc_fence_after();
        if (alive) {
            float *my = stage + (warp * 32) * STAGE_PITCH;
            for (int c0 = 0; c0 < p.outw; c0 += 32) {
                float v[32];
                tmem_ld32(tmem + ((uint32_t)(warp * 32) << 16) + (uint32_t)c0, v);
#pragma unroll
                for (int c = 0; c < 32; ++c) my[lane * STAGE_PITCH + c] = v[c];
                __syncwarp();
                const bool col_ok = c0 + lane < p.outw;
                float run = 0.f;
                int cur_row = -1;
                const int rend = min(32, rows - warp * 32);
                for (int r = 0; r < rend; ++r) {
                    int dst = s_scatter[warp * 32 + r];
                    float x = my[r * STAGE_PITCH + lane];
                    if (dst != cur_row) {
                        if (cur_row >= 0 && col_ok) atomicAdd(p.acc + (int64_t)cur_row * p.outw + c0 + lane, run);
                        cur_row = dst;
                        run = x;
                    } else {
                        run += x;
                    }
                }
                if (cur_row >= 0 && col_ok) atomicAdd(p.acc + (int64_t)cur_row * p.outw + c0 + lane, run);
                __syncwarp();
            }
        }
        tc_fence_before();
        __syncthreads();
    }
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, p.ncols);
}

struct VvorTcParams {
    const uint16_t *a, *b;  // (n_a, Ma), (n_b, Cb)
    const int32_t *a_idx, *b_idx;
    const int64_t *seg;
    const int32_t *cum;
    float *acc;             // (n_o, Ma, Cb)
    int n_o, Ma, Cb, fmt;
    uint32_t ncols;
};

__global__ void __launch_bounds__(128) vvor_tc_kernel(VvorTcParams p) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t s_bar;
    __shared__ uint32_t s_tmem;
    __shared__ int32_t s_ia[CH], s_ib[CH];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const int row_tiles = (p.Ma + 127) >> 7;
    const int ablk = row_tiles * 2;           // 64-channel blocks held for A (padded to 128 rows per tile)
    const int bblk = (p.Cb + 63) >> 6;
    const uint32_t a_tile = base;
    const uint32_t b_tile = a_tile + (uint32_t)ablk * BLK_BYTES;
    float *stage = reinterpret_cast<float *>(smem_raw + (b_tile + (uint32_t)bblk * BLK_BYTES - smem_u32(smem_raw)));
    const uint32_t bar = smem_u32(&s_bar);

    if (tid == 0) {
        mbar_init(bar, 1);
        fence_mbar_init();
    }
    if (warp == 0) tmem_alloc(smem_u32(&s_tmem), p.ncols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = s_tmem;

    const int total = p.cum[p.n_o];
    const int per = (total + gridDim.x - 1) / gridDim.x;
    const int lo = blockIdx.x * per, hi = min(total, lo + per);
    const uint32_t idesc = instr_desc(p.fmt, 128, p.Cb, 1, 1);
    uint32_t phase = 0;
    bool alive = true;
    bool fresh = true;  // next MMA starts a new accumulation
    ChunkCursor cur;
    if (lo < hi) cur.seek(p.cum, p.seg, p.n_o, lo);

    for (int chunk = lo; chunk < hi && alive; ++chunk) {
        cur.advance(p.cum, p.seg, p.n_o, chunk);
        const int o = cur.tap;
        const int64_t t0 = cur.first(chunk);
        const int rows = cur.rows(chunk);
        const bool last_of_tap = (chunk + 1 == hi) || cur.last_of_tap(chunk);
        if (tid < rows) {
            s_ia[tid] = p.a_idx[t0 + tid];
            s_ib[tid] = p.b_idx[t0 + tid];
        }
        __syncthreads();
        gather_tile<true>(a_tile, p.a, s_ia, rows, p.Ma, tid, 128);
        gather_tile<true>(b_tile, p.b, s_ib, rows, p.Cb, tid, 128);
        cp_async_wait_all();
        fence_async_smem();
        __syncthreads();

        if (tid == 0) {
            tc_fence_after();
            const int ksteps = (rows + 15) >> 4;
            for (int rt = 0; rt < row_tiles; ++rt) {
                for (int s = 0; s < ksteps; ++s) {
                    uint64_t ad = smem_desc(a_tile + (uint32_t)(rt * 2) * BLK_BYTES + (uint32_t)s * 2048, BLK_BYTES, 1024);
                    uint64_t bd = smem_desc(b_tile + (uint32_t)s * 2048, BLK_BYTES, 1024);
                    tc_mma(tmem + (uint32_t)(rt * p.Cb), ad, bd, idesc, (fresh && s == 0) ? 0u : 1u);
                }
            }
            tc_commit(bar);
        }
        fresh = false;
        alive = mbar_wait(bar, phase, 2u);
        phase ^= 1u;
        tc_fence_after();
        if (alive && last_of_tap) {
            float *my = stage + (warp * 32) * STAGE_PITCH;
            float *dst_o = p.acc + (int64_t)o * p.Ma * p.Cb;
            for (int rt = 0; rt < row_tiles; ++rt) {
                const int m_base = rt * 128 + warp * 32;
                for (int c0 = 0; c0 < p.Cb; c0 += 32) {
                    float v[32];
                    tmem_ld32(tmem + ((uint32_t)(warp * 32) << 16) + (uint32_t)(rt * p.Cb + c0), v);
#pragma unroll
                    for (int c = 0; c < 32; ++c) my[lane * STAGE_PITCH + c] = v[c];
                    __syncwarp();
                    if (c0 + lane < p.Cb) {
                        const int rend = min(32, p.Ma - m_base);
                        for (int r = 0; r < rend; ++r)
                            atomicAdd(dst_o + (int64_t)(m_base + r) * p.Cb + c0 + lane, my[r * STAGE_PITCH + lane]);
                    }
                    __syncwarp();
                }
            }
            fresh = true;
        }
        tc_fence_before();
        __syncthreads();
    }
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, p.ncols);
}

__global__ void transpose_weight_kernel(const uint16_t *__restrict__ w, uint16_t *__restrict__ wt, int K, int C, int M) {
    // wt[k][m][c] = w[k][c][m]
    __shared__ uint16_t tile[32][33];
    const int k = blockIdx.z;
    const int c0 = blockIdx.y * 32, m0 = blockIdx.x * 32;
    const uint16_t *src = w + (int64_t)k * C * M;
    uint16_t *dst = wt + (int64_t)k * C * M;
    for (int r = threadIdx.y; r < 32; r += blockDim.y) {
        int c = c0 + r, m = m0 + threadIdx.x;
        if (c < C && m < M) tile[r][threadIdx.x] = src[(int64_t)c * M + m];
    }
    __syncthreads();
    for (int r = threadIdx.y; r < 32; r += blockDim.y) {
        int m = m0 + r, c = c0 + threadIdx.x;
        if (c < C && m < M) dst[(int64_t)m * C + c] = tile[threadIdx.x][r];
    }
}

uint32_t pow2_cols(int n) {
    uint32_t c = 32;
    while ((int)c < n) c <<= 1;
    return c;
}

// CTAs per SM: bounded by shared memory (227 KiB usable, 1 KiB reserved per
// CTA), by TMEM (512 columns) and by registers / warp slots.
int ctas_per_sm(size_t smem, uint32_t ncols) {
    int by_smem = (int)((size_t)232448 / (smem + 1024));
    int by_tmem = (int)(512 / ncols);
    int occ = by_smem < by_tmem ? by_smem : by_tmem;
    if (occ > 8) occ = 8;
    return occ < 1 ? 1 : occ;
}

// Dynamic shared memory padded so that at most 512 / ncols CTAs share an SM
// (their TMEM allocations then always fit).
size_t pad_for_tmem(size_t smem, uint32_t ncols) {
    size_t max_ctas = 512 / ncols;
    size_t floor_bytes = (size_t)232448 / (max_ctas + 1) + 1024;
    return smem > floor_bytes ? smem : floor_bytes;
}

bool aligned16(const void *p) { return ((uintptr_t)p & 15) == 0; }

}  // namespace

bool mvmr_tensor_supported(const MvmrArgs &a) {
    if (a.dtype != PCX_F16 && a.dtype != PCX_BF16) return false;
    if (a.G != 1 || !a.seg_offs || a.T <= 0) return false;
    const int inw = a.transpose ? a.M : a.C, outw = a.transpose ? a.C : a.M;
    if (inw % 16 || outw % 16 || inw < 16 || outw < 16 || inw > 256 || outw > 256) return false;
    if (!aligned16(a.weight) || !aligned16(a.feat)) return false;
    if (a.T / CH + a.K >= INT32_MAX) return false;
    return true;
}

bool vvor_tensor_supported(const VvorArgs &a) {
    if (a.dtype != PCX_F16 && a.dtype != PCX_BF16) return false;
    if (a.G != 1 || !a.seg_offs || a.T <= 0) return false;
    if (a.Ma % 16 || a.Cb % 16 || a.Ma < 16 || a.Cb < 16 || a.Ma > 256 || a.Cb > 256) return false;
    if (((a.Ma + 127) / 128) * a.Cb > 512) return false;
    if (!aligned16(a.a) || !aligned16(a.b)) return false;
    if (a.n_o > 65536) return false;
    return true;
}

int mvmr_tensor(const MvmrArgs &a, cudaStream_t stream) {
    const int inw = a.transpose ? a.M : a.C, outw = a.transpose ? a.C : a.M;
    const uint16_t *bmat = (const uint16_t *)a.weight;
    if (!a.transpose) {  // forward: rows of the B tile are output channels -> (K, M, C)
        dim3 grid((a.M + 31) / 32, (a.C + 31) / 32, a.K), block(32, 8);
        transpose_weight_kernel<<<grid, block, 0, stream>>>((const uint16_t *)a.weight, (uint16_t *)a.weight_t, a.K, a.C, a.M);
        PCX_LAUNCH_CHECK();
        bmat = (const uint16_t *)a.weight_t;
    }
    chunk_table_kernel<<<1, 128, 0, stream>>>(a.seg_offs, a.K, CH, a.chunk_table);
    PCX_LAUNCH_CHECK();
    MvmrTcParams p;
    p.bmat = bmat, p.feat = (const uint16_t *)a.feat, p.gather = a.gather, p.scatter = a.scatter;
    p.seg = a.seg_offs, p.cum = a.chunk_table, p.acc = a.acc;
    p.K = a.K, p.inw = inw, p.outw = outw, p.fmt = a.dtype == PCX_BF16 ? 1 : 0;
    p.ncols = pow2_cols(outw);
    const int kb = (inw + 63) / 64;
    size_t smem = 1024 + (size_t)kb * BLK_BYTES + (size_t)kb * outw * 128 + (size_t)CH * STAGE_PITCH * 4;
    smem = pad_for_tmem(smem, p.ncols);
    if (smem > 232448 - 1024) PCX_FAIL(PCX_E_UNSUPPORTED, "mvmr tensor kernel does not fit (smem %zu)", smem);
    PCX_CUDA(cudaFuncSetAttribute(mvmr_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    PCX_CUDA(cudaFuncSetAttribute(mvmr_tc_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
    const int occ = ctas_per_sm(smem, p.ncols);
    int64_t upper = a.T / CH + a.K + 1;
    int64_t grid = std::min<int64_t>(upper, (int64_t)occ * num_sms());
    prof_begin(a.transpose ? "mvmr_tc_kernel(dgrad)" : "mvmr_tc_kernel(fwd)", stream);
    mvmr_tc_kernel<<<(unsigned)grid, 128, smem, stream>>>(p);
    prof_end(stream);
    PCX_LAUNCH_CHECK();
    return PCX_OK;
}

int vvor_tensor(const VvorArgs &a, cudaStream_t stream) {
    chunk_table_kernel<<<1, 128, 0, stream>>>(a.seg_offs, (int)a.n_o, CH, a.chunk_table);
    PCX_LAUNCH_CHECK();
    VvorTcParams p;
    p.a = (const uint16_t *)a.a, p.b = (const uint16_t *)a.b, p.a_idx = a.a_idx, p.b_idx = a.b_idx;
    p.seg = a.seg_offs, p.cum = a.chunk_table, p.acc = a.acc;
    p.n_o = (int)a.n_o, p.Ma = a.Ma, p.Cb = a.Cb, p.fmt = a.dtype == PCX_BF16 ? 1 : 0;
    const int row_tiles = (a.Ma + 127) / 128;
    p.ncols = pow2_cols(row_tiles * a.Cb);
    size_t smem = 1024 + (size_t)(row_tiles * 2) * BLK_BYTES + (size_t)((a.Cb + 63) / 64) * BLK_BYTES +
                  (size_t)CH * STAGE_PITCH * 4;
    smem = pad_for_tmem(smem, p.ncols);
    if (smem > 232448 - 1024) PCX_FAIL(PCX_E_UNSUPPORTED, "vvor tensor kernel does not fit (smem %zu)", smem);
    PCX_CUDA(cudaFuncSetAttribute(vvor_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    PCX_CUDA(cudaFuncSetAttribute(vvor_tc_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
    const int occ = ctas_per_sm(smem, p.ncols);
    int64_t upper = a.T / CH + a.n_o + 1;
    int64_t grid = std::min<int64_t>(upper, (int64_t)occ * num_sms());
    prof_begin("vvor_tc_kernel", stream);
    vvor_tc_kernel<<<(unsigned)grid, 128, smem, stream>>>(p);
    prof_end(stream);
    PCX_LAUNCH_CHECK();
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
