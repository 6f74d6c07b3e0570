// Fused layer normalisation over a ragged batch, with the residual add and the
// ReLU of a residual block folded into the same pass:
//
//   y = relu?( (x - mean_s) * rstd_s * weight + bias  (+ residual) )
//
// mean_s and rstd_s are the statistics of ALL elements (rows x channels) of
// sample s, computed in two passes exactly as the reference composes them
// (layers/norm.py:118-130: mean first, then the variance of the centred values,
// rstd = 1 / sqrt(var + eps)); the reference spends about a dozen elementwise
// and reduction launches on it, this file two reads of x from HBM forward (the
// statistics pass centres on block means while a block's rows are still cached
// and merges the blocks exactly) and two passes backward.  HBM-bound: bytes are
// what counts, the arithmetic is fp32.
//
// Backward, with g' = g masked by the ReLU, gh = g' * weight, xh = (x - mean) * rstd,
// n = rows_s * C:
//   dx = rstd * (gh - sum_s(gh) / n - xh * sum_s(gh * xh) / n)
//   dweight[c] = sum over rows of g' * xh,  dbias[c] = sum over rows of g',
//   dresidual = g'.
#include <cub/cub.cuh>

#include "rowwise.cuh"
#include "sparse_kernels.cuh"

namespace pcx {
namespace {

constexpr int LN_ROWS = 512;      // rows per block
constexpr int LN_THREADS = 256;

__device__ __forceinline__ float block_sum(float v, float *scratch) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float t = 0.f;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) t += scratch[w];
    return t;
}

__global__ void ln_tail_kernel(int64_t *offsets, int64_t S, int64_t total) {
    if (threadIdx.x == 0 && blockIdx.x == 0) offsets[S] = total;
}

// Row offsets of a batch of a few samples in one small launch: one warp scans 32 lengths at a time.
__global__ void ln_small_offsets_kernel(const int64_t *__restrict__ lengths, int64_t *offsets, int64_t S, int64_t total) {
    const int lane = threadIdx.x;
    int64_t carry = 0;
    for (int64_t base = 0; base < S; base += 32) {
        const int64_t v = base + lane < S ? lengths[base + lane] : 0;
        int64_t incl = v;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int64_t up = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += up;
        }
        if (base + lane < S) offsets[base + lane] = carry + incl - v;
        carry += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (lane == 0) offsets[S] = total;
}

// The kernels below share one shape: a block owns LN_ROWS consecutive rows, a thread
// keeps one vector column (VN channels, one 16-byte access when VN > 1) and walks the
// rows of its row lane.  `uniform` blocks lie inside one sample (all but S - 1 of them).
struct BlockRows {
    int64_t row0, row1, s_first;
    bool uniform;
    __device__ __forceinline__ BlockRows(const int64_t *__restrict__ offsets, int64_t N, int64_t S) {
        row0 = (int64_t)blockIdx.x * LN_ROWS;
        row1 = min(N, row0 + LN_ROWS);
        s_first = segment_of_row(offsets, S, row0);
        uniform = s_first == segment_of_row(offsets, S, row1 - 1);
    }
};

// Statistics of the layer norm with ONE read of x from HBM.  A block first sums its rows (block
// mean), then sums the squares centred on that mean while its rows are still in the caches, and
// leaves (count, mean, M2) per (block, sample) piece; ln_combine_kernel merges the pieces of a
// sample exactly (M2 = sum M2_p + n_p (mean_p - mean)^2), which keeps the accuracy of the
// two-pass formula.  The piece of sample s in block b is record b + s (pieces are ordered, and
// going to the next piece advances b or s by one), so a sample's pieces are consecutive records.
struct Moments { float n, mean, m2, pad; };

template <typename T, int VN>
__global__ void ln_moments_kernel(const T *__restrict__ x, const int64_t *__restrict__ offsets, Moments *rec,
                                  int64_t N, int64_t S, int C) {
    __shared__ float scratch[LN_THREADS / 32];
    const BlockRows B(offsets, N, S);
    const RowLayout L(C, VN);
    const int64_t s_last = B.uniform ? B.s_first : segment_of_row(offsets, S, B.row1 - 1);
    for (int64_t s = B.s_first; s <= s_last; ++s) {
        const int64_t lo = max(B.row0, offsets[s]), hi = min(B.row1, offsets[s + 1]);
        if (hi <= lo) continue;   // an empty sample inside the block (same decision in every thread)
        float mu = 0.f;
        float result[2];
#pragma unroll
        for (int pass = 0; pass < 2; ++pass) {
            float acc = 0.f;
            for (int cp = 0; cp * L.vcb < L.vc_total; ++cp) {
                const int vcol = cp * L.vcb + L.vc;
                if (vcol >= L.vc_total || L.lane >= L.lanes) continue;
#pragma unroll 4
                for (int64_t r = lo + L.lane; r < hi; r += L.lanes) {
                    float v[VN];
                    load_vec<T, VN>(x + r * C + (int64_t)vcol * VN, v);
#pragma unroll
                    for (int i = 0; i < VN; ++i) {
                        const float d = v[i] - mu;
                        acc += pass ? d * d : d;
                    }
                }
            }
            result[pass] = block_sum(acc, scratch);
            if (pass == 0) mu = result[0] / ((float)(hi - lo) * (float)C);
        }
        if (threadIdx.x == 0) rec[blockIdx.x + s] = Moments{(float)(hi - lo) * (float)C, mu, result[1], 0.f};
    }
}

// The same statistics with the block's rows held in registers (rows of at most 256 sixteen-byte
// columns): a thread loads MOM_R rows of its column once, and both sweeps -- the sum, then the squares
// centred on the block mean -- run over those registers.  A block covers MOM_R * (256 / columns) rows.
constexpr int MOM_R = 4;

template <typename T, int VN>
__global__ void __launch_bounds__(LN_THREADS) ln_moments_reg_kernel(const T *__restrict__ x, const int64_t *__restrict__ offsets,
                                                                    Moments *rec, int64_t N, int64_t S, int C, int mom_rows) {
    __shared__ float scratch[LN_THREADS / 32];
    const RowLayout L(C, VN);   // one pass: vc_total <= blockDim
    const int64_t row0 = (int64_t)blockIdx.x * mom_rows, row1 = min(N, row0 + mom_rows);
    const int64_t s_first = segment_of_row(offsets, S, row0), s_last = segment_of_row(offsets, S, row1 - 1);
    float v[MOM_R][VN];
    int64_t rows[MOM_R];
#pragma unroll
    for (int k = 0; k < MOM_R; ++k) {
        rows[k] = row0 + L.lane + (int64_t)k * L.lanes;
        if (L.lane < L.lanes && rows[k] < row1) {
            load_vec<T, VN>(x + rows[k] * C + (int64_t)L.vc * VN, v[k]);
        } else {
            rows[k] = -1;
#pragma unroll
            for (int i = 0; i < VN; ++i) v[k][i] = 0.f;
        }
    }
    for (int64_t s = s_first; s <= s_last; ++s) {
        const int64_t lo = max(row0, offsets[s]), hi = min(row1, offsets[s + 1]);
        if (hi <= lo) continue;   // an empty sample inside the block (same decision in every thread)
        float mu = 0.f, result[2];
#pragma unroll
        for (int pass = 0; pass < 2; ++pass) {
            float acc = 0.f;
#pragma unroll
            for (int k = 0; k < MOM_R; ++k) {
                if (rows[k] >= lo && rows[k] < hi) {
#pragma unroll
                    for (int i = 0; i < VN; ++i) {
                        const float d = v[k][i] - mu;
                        acc += pass ? d * d : d;
                    }
                }
            }
            result[pass] = block_sum(acc, scratch);
            if (pass == 0) mu = result[0] / ((float)(hi - lo) * (float)C);
        }
        if (threadIdx.x == 0) rec[blockIdx.x + s] = Moments{(float)(hi - lo) * (float)C, mu, result[1], 0.f};
    }
}

constexpr int COMBINE_THREADS = 256;

__device__ __forceinline__ double block_sum_f64(double v, double *scratch) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
    __syncthreads();
    double t = 0.0;
    for (int w = 0; w < COMBINE_THREADS / 32; ++w) t += scratch[w];
    return t;
}

// one block per sample: the sample's pieces are spread over the threads, the sums are folded in fp64
__global__ void __launch_bounds__(COMBINE_THREADS) ln_combine_kernel(const Moments *__restrict__ rec,
                                                                     const int64_t *__restrict__ offsets, float *mean,
                                                                     float *rstd, int64_t S, float eps, int mom_rows) {
    __shared__ double scratch[COMBINE_THREADS / 32];
    const int64_t s = blockIdx.x;
    const int64_t lo = offsets[s], hi = offsets[s + 1];
    if (hi <= lo) {   // the same decision in every thread
        if (threadIdx.x == 0) mean[s] = 0.f, rstd[s] = 1.f / sqrtf(eps);
        return;
    }
    const int64_t b0 = lo / mom_rows, b1 = (hi - 1) / mom_rows;
    double n = 0.0, sum = 0.0;
    for (int64_t b = b0 + threadIdx.x; b <= b1; b += COMBINE_THREADS) {
        const Moments m = rec[b + s];
        n += m.n, sum += (double)m.n * m.mean;
    }
    n = block_sum_f64(n, scratch);
    sum = block_sum_f64(sum, scratch);
    const double mu = sum / n;
    double m2 = 0.0;
    for (int64_t b = b0 + threadIdx.x; b <= b1; b += COMBINE_THREADS) {
        const Moments m = rec[b + s];
        const double d = (double)m.mean - mu;
        m2 += (double)m.m2 + (double)m.n * d * d;
    }
    m2 = block_sum_f64(m2, scratch);
    if (threadIdx.x == 0) mean[s] = (float)mu, rstd[s] = 1.f / sqrtf((float)(m2 / n) + eps);
}

template <typename T, int VN>
__global__ void __launch_bounds__(LN_THREADS, 5) ln_apply_kernel(const T *__restrict__ x, const int64_t *__restrict__ offsets,
                                const float *__restrict__ mean, const float *__restrict__ rstd,
                                const float *__restrict__ weight, const float *__restrict__ bias,
                                const T *__restrict__ residual, T *y, int64_t N, int64_t S, int C, int relu) {
    const BlockRows B(offsets, N, S);
    const RowLayout L(C, VN);
    for (int cp = 0; cp * L.vcb < L.vc_total; ++cp) {
        const int vcol = cp * L.vcb + L.vc;
        if (vcol >= L.vc_total || L.lane >= L.lanes) continue;
        float w[VN], b[VN];
#pragma unroll
        for (int i = 0; i < VN; ++i) {
            w[i] = weight ? weight[vcol * VN + i] : 1.f;
            b[i] = weight ? bias[vcol * VN + i] : 0.f;
        }
#pragma unroll 4
        for (int64_t r = B.row0 + L.lane; r < B.row1; r += L.lanes) {
            const int64_t s = B.uniform ? B.s_first : segment_of_row(offsets, S, r);
            const float mu = mean[s], rs = rstd[s];
            const int64_t at = r * C + (int64_t)vcol * VN;
            float v[VN], res[VN];
            load_vec<T, VN>(x + at, v);
            if (residual) load_vec<T, VN>(residual + at, res);
#pragma unroll
            for (int i = 0; i < VN; ++i) {
                float o = (v[i] - mu) * rs * w[i] + b[i];
                if (residual) o += res[i];
                v[i] = relu ? fmaxf(o, 0.f) : o;
            }
            store_vec<T, VN>(y + at, v);
        }
    }
}

// Per-sample sums of gh and gh * xh, per-channel sums of g' * xh and g', and
// (optionally) the masked gradient for the residual branch.  Per-sample partial sums
// stay in registers while a thread's rows belong to one sample; the per-channel sums of
// the row lanes are folded in shared memory, one atomic per channel and block.
template <typename T, int VN>
__global__ void __launch_bounds__(LN_THREADS, 4) ln_bwd_sums_kernel(const T *__restrict__ g, const T *__restrict__ x, const T *__restrict__ y,
                                   const int64_t *__restrict__ offsets, const float *__restrict__ mean,
                                   const float *__restrict__ rstd, const float *__restrict__ weight, float *s1,
                                   float *s2, float *dweight, float *dbias, T *dresidual, int64_t N, int64_t S,
                                   int C, int relu) {
    __shared__ float scratch[LN_THREADS / 32];
    __shared__ float col_w[LN_THREADS * VN], col_b[LN_THREADS * VN];
    const BlockRows B(offsets, N, S);
    const RowLayout L(C, VN);
    float a = 0.f, b = 0.f;     // running sums of gh and gh * xh for sample `cur`
    int64_t cur = B.s_first;
    for (int cp = 0; cp * L.vcb < L.vc_total; ++cp) {
        const int vcol = cp * L.vcb + L.vc;
        const bool active = vcol < L.vc_total && L.lane < L.lanes;
        float w[VN], dw[VN], db[VN];
#pragma unroll
        for (int i = 0; i < VN; ++i) {
            w[i] = (weight && active) ? weight[vcol * VN + i] : 1.f;
            dw[i] = db[i] = 0.f;
        }
        if (active) {
#pragma unroll 2
            for (int64_t r = B.row0 + L.lane; r < B.row1; r += L.lanes) {
                const int64_t s = B.uniform ? B.s_first : segment_of_row(offsets, S, r);
                if (s != cur) {
                    atomicAdd(s1 + cur, a);
                    atomicAdd(s2 + cur, b);
                    a = b = 0.f;
                    cur = s;
                }
                const float mu = mean[s], rs = rstd[s];
                const int64_t at = r * C + (int64_t)vcol * VN;
                float gv[VN], xv[VN], yv[VN];
                load_vec<T, VN>(g + at, gv);
                load_vec<T, VN>(x + at, xv);
                if (relu) load_vec<T, VN>(y + at, yv);
#pragma unroll
                for (int i = 0; i < VN; ++i) {
                    if (relu && !(yv[i] > 0.f)) gv[i] = 0.f;
                    const float xh = (xv[i] - mu) * rs;
                    a += gv[i] * w[i];
                    b += gv[i] * w[i] * xh;
                    dw[i] += gv[i] * xh;
                    db[i] += gv[i];
                }
                if (dresidual) store_vec<T, VN>(dresidual + at, gv);
            }
        }
        if (dweight) {
            // col_*[lane][column of the pass]: fold the row lanes, then one atomic per channel
#pragma unroll
            for (int i = 0; i < VN; ++i) {
                col_w[(L.lane * L.vcb + L.vc) * VN + i] = dw[i];
                col_b[(L.lane * L.vcb + L.vc) * VN + i] = db[i];
            }
            __syncthreads();
            const int cols = L.vcb * VN;
            for (int t = threadIdx.x; t < cols; t += LN_THREADS) {
                const int c = cp * cols + t;
                if (c < C) {
                    float tw = 0.f, tb = 0.f;
                    for (int q = 0; q < L.lanes; ++q) tw += col_w[q * cols + t], tb += col_b[q * cols + t];
                    atomicAdd(dweight + c, tw);
                    atomicAdd(dbias + c, tb);
                }
            }
            __syncthreads();
        }
    }
    if (B.uniform) {
        a = block_sum(a, scratch);
        b = block_sum(b, scratch);
        if (threadIdx.x == 0) {
            atomicAdd(s1 + B.s_first, a);
            atomicAdd(s2 + B.s_first, b);
        }
    } else {
        atomicAdd(s1 + cur, a);
        atomicAdd(s2 + cur, b);
    }
}

template <typename T, int VN>
__global__ void ln_bwd_apply_kernel(const T *__restrict__ g, const T *__restrict__ x, const T *__restrict__ y,
                                    const int64_t *__restrict__ offsets, const float *__restrict__ mean,
                                    const float *__restrict__ rstd, const float *__restrict__ weight,
                                    const float *__restrict__ s1, const float *__restrict__ s2, T *dx, int64_t N,
                                    int64_t S, int C, int relu) {
    const BlockRows B(offsets, N, S);
    const RowLayout L(C, VN);
    for (int cp = 0; cp * L.vcb < L.vc_total; ++cp) {
        const int vcol = cp * L.vcb + L.vc;
        if (vcol >= L.vc_total || L.lane >= L.lanes) continue;
        float w[VN];
#pragma unroll
        for (int i = 0; i < VN; ++i) w[i] = weight ? weight[vcol * VN + i] : 1.f;
#pragma unroll 2
        for (int64_t r = B.row0 + L.lane; r < B.row1; r += L.lanes) {
            const int64_t s = B.uniform ? B.s_first : segment_of_row(offsets, S, r);
            const float mu = mean[s], rs = rstd[s];
            const float inv_n = 1.f / ((float)(offsets[s + 1] - offsets[s]) * (float)C);
            const float m1 = s1[s] * inv_n, m2 = s2[s] * inv_n;
            const int64_t at = r * C + (int64_t)vcol * VN;
            float gv[VN], xv[VN], yv[VN];
            load_vec<T, VN>(g + at, gv);   // with relu == 0 this may be the gradient the sums pass already masked
            load_vec<T, VN>(x + at, xv);
            if (relu) load_vec<T, VN>(y + at, yv);
#pragma unroll
            for (int i = 0; i < VN; ++i) {
                if (relu && !(yv[i] > 0.f)) gv[i] = 0.f;
                const float xh = (xv[i] - mu) * rs;
                gv[i] = rs * (gv[i] * w[i] - m1 - xh * m2);
            }
            store_vec<T, VN>(dx + at, gv);
        }
    }
}

// ---------------------------------------------------------------- grouped statistics ----
// Group and instance normalisation: the statistics of sample s are kept per channel group g
// (G groups of W = C / G consecutive channels; instance norm is W = 1) in arrays indexed
// s * G + g.  Same block shape as above; a thread's VN channels may fall into different groups,
// so every channel keeps its own running sum.  Blocks inside one sample fold their sums per
// group in shared memory (G floats) and issue one atomic per group; blocks that straddle a
// sample boundary use per-thread atomics.
struct GroupStats {
    float mu[8], rs[8];
    int64_t at = -1;
    template <int VN>
    __device__ __forceinline__ void load(const float *__restrict__ mean, const float *__restrict__ rstd, int64_t s,
                                         int G, const int *g) {
        if (s == at) return;
        at = s;
#pragma unroll
        for (int i = 0; i < VN; ++i) {
            mu[i] = mean ? mean[s * G + g[i]] : 0.f;
            rs[i] = rstd ? rstd[s * G + g[i]] : 1.f;
        }
    }
};

template <int VN>
__device__ __forceinline__ void flush_groups(float *dst, const int *g, float *v) {
#pragma unroll
    for (int i = 0; i < VN; ++i) {
        if (v[i] != 0.f) atomicAdd(dst + g[i], v[i]);
        v[i] = 0.f;
    }
}

// sums[s * G + g] += sum of x (mean == null) or of (x - mean)^2
template <typename T, int VN>
__global__ void gn_sum_kernel(const T *__restrict__ x, const int64_t *__restrict__ offsets,
                              const float *__restrict__ mean, float *sums, int64_t N, int64_t S, int C, int G) {
    extern __shared__ float s_grp[];
    const BlockRows B(offsets, N, S);
    const RowLayout L(C, VN);
    const int W = C / G;
    if (B.uniform) {
        for (int t = threadIdx.x; t < G; t += blockDim.x) s_grp[t] = 0.f;
        __syncthreads();
    }
    for (int cp = 0; cp * L.vcb < L.vc_total; ++cp) {
        const int vcol = cp * L.vcb + L.vc;
        if (vcol >= L.vc_total || L.lane >= L.lanes) continue;
        int g[VN];
        float acc[VN];
#pragma unroll
        for (int i = 0; i < VN; ++i) g[i] = (vcol * VN + i) / W, acc[i] = 0.f;
        GroupStats st;
        int64_t cur = B.s_first;
#pragma unroll 2
        for (int64_t r = B.row0 + L.lane; r < B.row1; r += L.lanes) {
            const int64_t s = B.uniform ? B.s_first : segment_of_row(offsets, S, r);
            if (s != cur) {
                flush_groups<VN>(sums + cur * G, g, acc);
                cur = s;
            }
            st.load<VN>(mean, nullptr, s, G, g);
            float v[VN];
            load_vec<T, VN>(x + r * C + (int64_t)vcol * VN, v);
#pragma unroll
            for (int i = 0; i < VN; ++i) {
                const float d = v[i] - st.mu[i];
                acc[i] += mean ? d * d : d;
            }
        }
        flush_groups<VN>(B.uniform ? s_grp : sums + cur * G, g, acc);
    }
    if (B.uniform) {
        __syncthreads();
        for (int t = threadIdx.x; t < G; t += blockDim.x)
            if (s_grp[t] != 0.f) atomicAdd(sums + B.s_first * G + t, s_grp[t]);
    }
}

__global__ void gn_stats_kernel(const float *__restrict__ sums, const int64_t *__restrict__ offsets, float *mean,
                                float *rstd, int64_t S, int G, int W, float eps, int second) {
    const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= S * G) return;
    const int64_t s = t / G, len = offsets[s + 1] - offsets[s];
    const float n = (float)(len > 0 ? len : 1) * (float)W;
    if (!second) mean[t] = sums[t] / n;
    else rstd[t] = 1.f / sqrtf(sums[t] / n + eps);
}

template <typename T, int VN>
__global__ void gn_apply_kernel(const T *__restrict__ x, const int64_t *__restrict__ offsets,
                                const float *__restrict__ mean, const float *__restrict__ rstd,
                                const float *__restrict__ weight, const float *__restrict__ bias, T *y, int64_t N,
                                int64_t S, int C, int G) {
    const BlockRows B(offsets, N, S);
    const RowLayout L(C, VN);
    const int W = C / G;
    for (int cp = 0; cp * L.vcb < L.vc_total; ++cp) {
        const int vcol = cp * L.vcb + L.vc;
        if (vcol >= L.vc_total || L.lane >= L.lanes) continue;
        int g[VN];
        float w[VN], b[VN];
#pragma unroll
        for (int i = 0; i < VN; ++i) {
            g[i] = (vcol * VN + i) / W;
            w[i] = weight ? weight[vcol * VN + i] : 1.f;
            b[i] = weight ? bias[vcol * VN + i] : 0.f;
        }
        GroupStats st;
#pragma unroll 2
        for (int64_t r = B.row0 + L.lane; r < B.row1; r += L.lanes) {
            const int64_t s = B.uniform ? B.s_first : segment_of_row(offsets, S, r);
            st.load<VN>(mean, rstd, s, G, g);
            const int64_t at = r * C + (int64_t)vcol * VN;
            float v[VN];
            load_vec<T, VN>(x + at, v);
#pragma unroll
            for (int i = 0; i < VN; ++i) v[i] = (v[i] - st.mu[i]) * st.rs[i] * w[i] + b[i];
            store_vec<T, VN>(y + at, v);
        }
    }
}

// Backward of the grouped norms, with gh = g * weight, xh = (x - mean) * rstd, n = rows_s * W:
//   dx = rstd * (gh - sum_{s,g}(gh) / n - xh * sum_{s,g}(gh * xh) / n),
//   dweight[c] = sum over rows of g * xh, dbias[c] = sum over rows of g.
template <typename T, int VN>
__global__ void gn_bwd_sums_kernel(const T *__restrict__ g_out, const T *__restrict__ x,
                                   const int64_t *__restrict__ offsets, const float *__restrict__ mean,
                                   const float *__restrict__ rstd, const float *__restrict__ weight, float *s1,
                                   float *s2, float *dweight, float *dbias, int64_t N, int64_t S, int C, int G) {
    extern __shared__ float s_grp[];   // 2 G: sums of gh, sums of gh * xh
    __shared__ float col_w[LN_THREADS * VN], col_b[LN_THREADS * VN];
    const BlockRows B(offsets, N, S);
    const RowLayout L(C, VN);
    const int W = C / G;
    if (B.uniform) {
        for (int t = threadIdx.x; t < 2 * G; t += blockDim.x) s_grp[t] = 0.f;
        __syncthreads();
    }
    for (int cp = 0; cp * L.vcb < L.vc_total; ++cp) {
        const int vcol = cp * L.vcb + L.vc;
        const bool active = vcol < L.vc_total && L.lane < L.lanes;
        int g[VN];
        float w[VN], a[VN], b[VN], dw[VN], db[VN];
#pragma unroll
        for (int i = 0; i < VN; ++i) {
            g[i] = active ? (vcol * VN + i) / W : 0;
            w[i] = (weight && active) ? weight[vcol * VN + i] : 1.f;
            a[i] = b[i] = dw[i] = db[i] = 0.f;
        }
        GroupStats st;
        int64_t cur = B.s_first;
#pragma unroll 2
        for (int64_t r = B.row0 + L.lane; active && r < B.row1; r += L.lanes) {
            const int64_t s = B.uniform ? B.s_first : segment_of_row(offsets, S, r);
            if (s != cur) {
                flush_groups<VN>(s1 + cur * G, g, a);
                flush_groups<VN>(s2 + cur * G, g, b);
                cur = s;
            }
            st.load<VN>(mean, rstd, s, G, g);
            const int64_t at = r * C + (int64_t)vcol * VN;
            float gv[VN], xv[VN];
            load_vec<T, VN>(g_out + at, gv);
            load_vec<T, VN>(x + at, xv);
#pragma unroll
            for (int i = 0; i < VN; ++i) {
                const float xh = (xv[i] - st.mu[i]) * st.rs[i];
                a[i] += gv[i] * w[i];
                b[i] += gv[i] * w[i] * xh;
                dw[i] += gv[i] * xh;
                db[i] += gv[i];
            }
        }
        flush_groups<VN>(B.uniform ? s_grp : s1 + cur * G, g, a);
        flush_groups<VN>(B.uniform ? s_grp + G : s2 + cur * G, g, b);
        if (dweight) {   // fold the row lanes in shared memory, then one atomic per channel and block
#pragma unroll
            for (int i = 0; i < VN; ++i) {
                col_w[(L.lane * L.vcb + L.vc) * VN + i] = dw[i];
                col_b[(L.lane * L.vcb + L.vc) * VN + i] = db[i];
            }
            __syncthreads();
            const int cols = L.vcb * VN;
            for (int t = threadIdx.x; t < cols; t += LN_THREADS) {
                const int c = cp * cols + t;
                if (c < C) {
                    float tw = 0.f, tb = 0.f;
                    for (int q = 0; q < L.lanes; ++q) tw += col_w[q * cols + t], tb += col_b[q * cols + t];
                    atomicAdd(dweight + c, tw);
                    atomicAdd(dbias + c, tb);
                }
            }
            __syncthreads();
        }
    }
    if (B.uniform) {
        __syncthreads();
        for (int t = threadIdx.x; t < G; t += blockDim.x) {
            if (s_grp[t] != 0.f) atomicAdd(s1 + B.s_first * G + t, s_grp[t]);
            if (s_grp[G + t] != 0.f) atomicAdd(s2 + B.s_first * G + t, s_grp[G + t]);
        }
    }
}

template <typename T, int VN>
__global__ void gn_bwd_apply_kernel(const T *__restrict__ g_out, const T *__restrict__ x,
                                    const int64_t *__restrict__ offsets, const float *__restrict__ mean,
                                    const float *__restrict__ rstd, const float *__restrict__ weight,
                                    const float *__restrict__ s1, const float *__restrict__ s2, T *dx, int64_t N,
                                    int64_t S, int C, int G) {
    const BlockRows B(offsets, N, S);
    const RowLayout L(C, VN);
    const int W = C / G;
    for (int cp = 0; cp * L.vcb < L.vc_total; ++cp) {
        const int vcol = cp * L.vcb + L.vc;
        if (vcol >= L.vc_total || L.lane >= L.lanes) continue;
        int g[VN];
        float w[VN], m1[VN], m2[VN];
#pragma unroll
        for (int i = 0; i < VN; ++i) g[i] = (vcol * VN + i) / W, w[i] = weight ? weight[vcol * VN + i] : 1.f;
        GroupStats st;
        int64_t have = -1;
#pragma unroll 2
        for (int64_t r = B.row0 + L.lane; r < B.row1; r += L.lanes) {
            const int64_t s = B.uniform ? B.s_first : segment_of_row(offsets, S, r);
            st.load<VN>(mean, rstd, s, G, g);
            if (s != have) {
                have = s;
                const float inv_n = 1.f / ((float)(offsets[s + 1] - offsets[s]) * (float)W);
#pragma unroll
                for (int i = 0; i < VN; ++i) m1[i] = s1[s * G + g[i]] * inv_n, m2[i] = s2[s * G + g[i]] * inv_n;
            }
            const int64_t at = r * C + (int64_t)vcol * VN;
            float gv[VN], xv[VN];
            load_vec<T, VN>(g_out + at, gv);
            load_vec<T, VN>(x + at, xv);
#pragma unroll
            for (int i = 0; i < VN; ++i) {
                const float xh = (xv[i] - st.mu[i]) * st.rs[i];
                gv[i] = st.rs[i] * (gv[i] * w[i] - m1[i] - xh * m2[i]);
            }
            store_vec<T, VN>(dx + at, gv);
        }
    }
}

struct LnWs {
    int64_t *offsets;
    Moments *rec;  // per (block, sample) piece of the forward statistics (layer norm only)
    float *sums;   // 2 * S
    void *cub_tmp;
    size_t cub_bytes;
};

size_t carve_ln(void *ws, int64_t S, LnWs *out, int64_t pieces = 0) {
    Carver c(ws);
    LnWs w;
    w.offsets = c.take<int64_t>((size_t)S + 1);
    w.rec = c.take<Moments>((size_t)pieces);
    w.sums = c.take<float>((size_t)2 * S + 1);
    size_t bytes = 0;
    cub::DeviceScan::ExclusiveSum(nullptr, bytes, (const int64_t *)nullptr, (int64_t *)nullptr, (int)std::max<int64_t>(S, 1));
    w.cub_bytes = bytes;
    w.cub_tmp = c.take<char>(bytes);
    if (out) *out = w;
    return c.off;
}

int ln_offsets(const int64_t *d_lengths, int64_t S, int64_t N, const LnWs &w, cudaStream_t stream) {
    if (S <= 4096) {
        ln_small_offsets_kernel<<<1, 32, 0, stream>>>(d_lengths, w.offsets, S, N);
        PCX_LAUNCH_CHECK();
        return PCX_OK;
    }
    size_t bytes = w.cub_bytes;
    PCX_CUDA(cub::DeviceScan::ExclusiveSum(w.cub_tmp, bytes, d_lengths, w.offsets, (int)S, stream));
    ln_tail_kernel<<<1, 32, 0, stream>>>(w.offsets, S, N);
    PCX_LAUNCH_CHECK();
    return PCX_OK;
}

// (block, sample) pieces of N rows in S samples: record b + s, b < blocks, s < S
// an upper bound for every block height the statistics pass may choose (at least MOM_R rows per block)
int64_t ln_pieces(int64_t N, int64_t S) { return (N + MOM_R - 1) / MOM_R + S; }

bool ln_sizes_ok(int64_t N, int64_t S, int C, int dtype) {
    return N >= 0 && S > 0 && S <= INT32_MAX && C > 0 && (dtype == PCX_F32 || dtype == PCX_F16 || dtype == PCX_BF16);
}

// CALL sees T (element type) and VN (channels per access: 16 bytes' worth when `vec`, else 1)
#define PCX_LN_DISPATCH(dtype, vec, CALL)                                                        \
    do {                                                                                         \
        if ((dtype) == PCX_F32) { using T = float; if (vec) { constexpr int VN = 4; CALL; } else { constexpr int VN = 1; CALL; } }           \
        else if ((dtype) == PCX_F16) { using T = __half; if (vec) { constexpr int VN = 8; CALL; } else { constexpr int VN = 1; CALL; } }      \
        else { using T = __nv_bfloat16; if (vec) { constexpr int VN = 8; CALL; } else { constexpr int VN = 1; CALL; } }                       \
    } while (0)

}  // namespace
}  // namespace pcx

using namespace pcx;

extern "C" {

size_t pcx_ragged_layer_norm_workspace_bytes(int64_t N, int64_t S) {
    return (S <= 0 || N < 0) ? 0 : carve_ln(nullptr, S, nullptr, ln_pieces(N, S));
}

int pcx_ragged_layer_norm(const void *d_x, const int64_t *d_lengths, const float *d_weight, const float *d_bias,
                          const void *d_residual, void *d_y, float *d_mean, float *d_rstd, int64_t N, int64_t S, int C,
                          double eps, int relu, int dtype, void *d_ws, size_t ws_bytes, void *stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    if (!ln_sizes_ok(N, S, C, dtype)) PCX_FAIL(PCX_E_ARG, "pcx_ragged_layer_norm: bad sizes or dtype");
    if (!d_lengths || !d_mean || !d_rstd || !d_ws || (N > 0 && (!d_x || !d_y)) || ((d_weight == nullptr) != (d_bias == nullptr)))
        PCX_FAIL(PCX_E_ARG, "pcx_ragged_layer_norm: null pointer (weight and bias come together)");
    if ((uintptr_t)d_ws % 256) PCX_FAIL(PCX_E_ALIGN, "pcx_ragged_layer_norm: workspace must be 256-byte aligned");
    LnWs w;
    size_t need = carve_ln(d_ws, S, &w, ln_pieces(N, S));
    if (ws_bytes < need) PCX_FAIL(PCX_E_CAPACITY, "pcx_ragged_layer_norm: workspace %zu < %zu bytes", ws_bytes, need);
    if (int rc = ln_offsets(d_lengths, S, N, w, stream)) return rc;
    const unsigned grid = (unsigned)((N + LN_ROWS - 1) / LN_ROWS);
    const bool vec = vec_ok(C, dtype, {d_x, d_y, d_residual});
    int mom_rows = LN_ROWS;
    const int vcols = C / (16 / (int)elem_size(dtype));   // sixteen-byte columns of a row (when vectorised)
    if (vec && vcols <= LN_THREADS) mom_rows = MOM_R * (LN_THREADS / vcols);   // rows held in registers
    if (N > 0) {
        if (mom_rows != LN_ROWS) {
            const unsigned mgrid = (unsigned)((N + mom_rows - 1) / mom_rows);
            PCX_LN_DISPATCH(dtype, true, (ln_moments_reg_kernel<T, VN><<<mgrid, LN_THREADS, 0, stream>>>((const T *)d_x, w.offsets, w.rec, N, S, C, mom_rows)));
        } else {
            PCX_LN_DISPATCH(dtype, vec, (ln_moments_kernel<T, VN><<<grid, LN_THREADS, 0, stream>>>((const T *)d_x, w.offsets, w.rec, N, S, C)));
        }
        PCX_LAUNCH_CHECK();
    }
    ln_combine_kernel<<<(unsigned)S, COMBINE_THREADS, 0, stream>>>(w.rec, w.offsets, d_mean, d_rstd, S, (float)eps, mom_rows);
    PCX_LAUNCH_CHECK();
    if (N > 0) {
        prof_begin("ln_apply_kernel", stream);
        PCX_LN_DISPATCH(dtype, vec, (ln_apply_kernel<T, VN><<<grid, LN_THREADS, 0, stream>>>(
                                   (const T *)d_x, w.offsets, d_mean, d_rstd, d_weight, d_bias, (const T *)d_residual,
                                   (T *)d_y, N, S, C, relu)));
        prof_end(stream);
        PCX_LAUNCH_CHECK();
    }
    return PCX_OK;
}

int pcx_ragged_layer_norm_backward(const void *d_grad_y, const void *d_x, const void *d_y, const int64_t *d_lengths,
                                   const float *d_weight, const float *d_mean, const float *d_rstd, void *d_grad_x,
                                   float *d_grad_weight, float *d_grad_bias, void *d_grad_residual, int64_t N,
                                   int64_t S, int C, int relu, int dtype, void *d_ws, size_t ws_bytes, void *stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    if (!ln_sizes_ok(N, S, C, dtype)) PCX_FAIL(PCX_E_ARG, "pcx_ragged_layer_norm_backward: bad sizes or dtype");
    if (!d_lengths || !d_mean || !d_rstd || !d_ws || (N > 0 && (!d_grad_y || !d_x || !d_grad_x)) || (relu && N > 0 && !d_y) ||
        ((d_grad_weight == nullptr) != (d_grad_bias == nullptr)))
        PCX_FAIL(PCX_E_ARG, "pcx_ragged_layer_norm_backward: null pointer");
    if ((uintptr_t)d_ws % 256) PCX_FAIL(PCX_E_ALIGN, "pcx_ragged_layer_norm_backward: workspace must be 256-byte aligned");
    LnWs w;
    size_t need = carve_ln(d_ws, S, &w);
    if (ws_bytes < need) PCX_FAIL(PCX_E_CAPACITY, "pcx_ragged_layer_norm_backward: workspace %zu < %zu bytes", ws_bytes, need);
    if (int rc = ln_offsets(d_lengths, S, N, w, stream)) return rc;
    PCX_CUDA(cudaMemsetAsync(w.sums, 0, (size_t)2 * S * sizeof(float), stream));
    if (d_grad_weight) {
        PCX_CUDA(cudaMemsetAsync(d_grad_weight, 0, (size_t)C * sizeof(float), stream));
        PCX_CUDA(cudaMemsetAsync(d_grad_bias, 0, (size_t)C * sizeof(float), stream));
    }
    if (N == 0) return PCX_OK;
    const unsigned grid = (unsigned)((N + LN_ROWS - 1) / LN_ROWS);
    const bool vec = vec_ok(C, dtype, {d_grad_y, d_x, d_y, d_grad_x, d_grad_residual});
    PCX_LN_DISPATCH(dtype, vec, (ln_bwd_sums_kernel<T, VN><<<grid, LN_THREADS, 0, stream>>>(
                               (const T *)d_grad_y, (const T *)d_x, (const T *)d_y, w.offsets, d_mean, d_rstd, d_weight,
                               w.sums, w.sums + S, d_grad_weight, d_grad_bias, (T *)d_grad_residual, N, S, C, relu)));
    PCX_LAUNCH_CHECK();
    // the sums pass wrote the ReLU-masked gradient as the residual's gradient: the second pass reads
    // that instead of masking again, which spares it the read of y
    const bool masked = relu && d_grad_residual;
    PCX_LN_DISPATCH(dtype, vec, (ln_bwd_apply_kernel<T, VN><<<grid, LN_THREADS, 0, stream>>>(
                               (const T *)(masked ? d_grad_residual : d_grad_y), (const T *)d_x, (const T *)d_y, w.offsets,
                               d_mean, d_rstd, d_weight, w.sums, w.sums + S, (T *)d_grad_x, N, S, C, masked ? 0 : relu)));
    PCX_LAUNCH_CHECK();
    return PCX_OK;
}

size_t pcx_ragged_group_norm_workspace_bytes(int64_t S, int G) {
    return (S <= 0 || G <= 0 || S * (int64_t)G > INT32_MAX) ? 0 : carve_ln(nullptr, S * G, nullptr);
}

int pcx_ragged_group_norm(const void *d_x, const int64_t *d_lengths, const float *d_weight, const float *d_bias,
                          void *d_y, float *d_mean, float *d_rstd, int64_t N, int64_t S, int C, int G, double eps,
                          int dtype, void *d_ws, size_t ws_bytes, void *stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    if (!ln_sizes_ok(N, S, C, dtype) || G <= 0 || C % G || S * (int64_t)G > INT32_MAX || G > 8192)
        PCX_FAIL(PCX_E_ARG, "pcx_ragged_group_norm: bad sizes or dtype (C must be a multiple of G <= 8192)");
    if (!d_lengths || !d_mean || !d_rstd || !d_ws || (N > 0 && (!d_x || !d_y)) || ((d_weight == nullptr) != (d_bias == nullptr)))
        PCX_FAIL(PCX_E_ARG, "pcx_ragged_group_norm: null pointer (weight and bias come together)");
    if ((uintptr_t)d_ws % 256) PCX_FAIL(PCX_E_ALIGN, "pcx_ragged_group_norm: workspace must be 256-byte aligned");
    const int64_t SG = S * G;
    LnWs w;
    size_t need = carve_ln(d_ws, SG, &w);
    if (ws_bytes < need) PCX_FAIL(PCX_E_CAPACITY, "pcx_ragged_group_norm: workspace %zu < %zu bytes", ws_bytes, need);
    if (int rc = ln_offsets(d_lengths, S, N, w, stream)) return rc;
    PCX_CUDA(cudaMemsetAsync(w.sums, 0, (size_t)2 * SG * sizeof(float), stream));
    const unsigned grid = (unsigned)((N + LN_ROWS - 1) / LN_ROWS), sgrid = (unsigned)((SG + 127) / 128);
    const bool vec = vec_ok(C, dtype, {d_x, d_y});
    const size_t smem = (size_t)G * sizeof(float);
    const int W = C / G;
    for (int second = 0; second < 2; ++second) {
        if (N > 0) {
            PCX_LN_DISPATCH(dtype, vec, (gn_sum_kernel<T, VN><<<grid, LN_THREADS, smem, stream>>>(
                                       (const T *)d_x, w.offsets, second ? d_mean : nullptr, w.sums + second * SG, N, S, C, G)));
            PCX_LAUNCH_CHECK();
        }
        gn_stats_kernel<<<sgrid, 128, 0, stream>>>(w.sums + second * SG, w.offsets, d_mean, d_rstd, S, G, W, (float)eps, second);
        PCX_LAUNCH_CHECK();
    }
    if (N > 0) {
        prof_begin("gn_apply_kernel", stream);
        PCX_LN_DISPATCH(dtype, vec, (gn_apply_kernel<T, VN><<<grid, LN_THREADS, 0, stream>>>(
                                   (const T *)d_x, w.offsets, d_mean, d_rstd, d_weight, d_bias, (T *)d_y, N, S, C, G)));
        prof_end(stream);
        PCX_LAUNCH_CHECK();
    }
    return PCX_OK;
}

int pcx_ragged_group_norm_backward(const void *d_grad_y, const void *d_x, const int64_t *d_lengths,
                                   const float *d_weight, const float *d_mean, const float *d_rstd, void *d_grad_x,
                                   float *d_grad_weight, float *d_grad_bias, int64_t N, int64_t S, int C, int G,
                                   int dtype, void *d_ws, size_t ws_bytes, void *stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    if (!ln_sizes_ok(N, S, C, dtype) || G <= 0 || C % G || S * (int64_t)G > INT32_MAX || G > 4096)
        PCX_FAIL(PCX_E_ARG, "pcx_ragged_group_norm_backward: bad sizes or dtype (C must be a multiple of G <= 4096)");
    if (!d_lengths || !d_mean || !d_rstd || !d_ws || (N > 0 && (!d_grad_y || !d_x || !d_grad_x)) ||
        ((d_grad_weight == nullptr) != (d_grad_bias == nullptr)))
        PCX_FAIL(PCX_E_ARG, "pcx_ragged_group_norm_backward: null pointer");
    if ((uintptr_t)d_ws % 256) PCX_FAIL(PCX_E_ALIGN, "pcx_ragged_group_norm_backward: workspace must be 256-byte aligned");
    const int64_t SG = S * G;
    LnWs w;
    size_t need = carve_ln(d_ws, SG, &w);
    if (ws_bytes < need) PCX_FAIL(PCX_E_CAPACITY, "pcx_ragged_group_norm_backward: workspace %zu < %zu bytes", ws_bytes, need);
    if (int rc = ln_offsets(d_lengths, S, N, w, stream)) return rc;
    PCX_CUDA(cudaMemsetAsync(w.sums, 0, (size_t)2 * SG * sizeof(float), stream));
    if (d_grad_weight) {
        PCX_CUDA(cudaMemsetAsync(d_grad_weight, 0, (size_t)C * sizeof(float), stream));
        PCX_CUDA(cudaMemsetAsync(d_grad_bias, 0, (size_t)C * sizeof(float), stream));
    }
    if (N == 0) return PCX_OK;
    const unsigned grid = (unsigned)((N + LN_ROWS - 1) / LN_ROWS);
    const bool vec = vec_ok(C, dtype, {d_grad_y, d_x, d_grad_x});
    PCX_LN_DISPATCH(dtype, vec, (gn_bwd_sums_kernel<T, VN><<<grid, LN_THREADS, (size_t)2 * G * sizeof(float), stream>>>(
                               (const T *)d_grad_y, (const T *)d_x, w.offsets, d_mean, d_rstd, d_weight, w.sums, w.sums + SG,
                               d_grad_weight, d_grad_bias, N, S, C, G)));
    PCX_LAUNCH_CHECK();
    PCX_LN_DISPATCH(dtype, vec, (gn_bwd_apply_kernel<T, VN><<<grid, LN_THREADS, 0, stream>>>(
                               (const T *)d_grad_y, (const T *)d_x, w.offsets, d_mean, d_rstd, d_weight, w.sums, w.sums + SG,
                               (T *)d_grad_x, N, S, C, G)));
    PCX_LAUNCH_CHECK();
    return PCX_OK;
}

}  // extern "C"
