// Fused layer normalisation over a ragged batch, with the residual add and the
// ReLU of a residual block folded into the same pass:
//
//   y = relu?( (x - mean_s) * rstd_s * weight + bias  (+ residual) )
//
// mean_s and rstd_s are the statistics of ALL elements (rows x channels) of
// sample s, computed in two passes exactly as the reference composes them
// (layers/norm.py:118-130: mean first, then the variance of the centred values,
// rstd = 1 / sqrt(var + eps)); the reference spends about a dozen elementwise
// and reduction launches on it, this file three passes over x forward and two
// backward.  HBM-bound: bytes are what counts, the arithmetic is fp32.
//
// Backward, with g' = g masked by the ReLU, gh = g' * weight, xh = (x - mean) * rstd,
// n = rows_s * C:
//   dx = rstd * (gh - sum_s(gh) / n - xh * sum_s(gh * xh) / n)
//   dweight[c] = sum over rows of g' * xh,  dbias[c] = sum over rows of g',
//   dresidual = g'.
#include <cub/cub.cuh>

#include "sparse_kernels.cuh"

namespace pcx {
namespace {

constexpr int LN_ROWS = 256;      // rows per block
constexpr int LN_THREADS = 256;

__device__ __forceinline__ int64_t sample_of(const int64_t *__restrict__ offsets, int64_t S, int64_t row) {
    int64_t lo = 0, hi = S;
    while (lo < hi) {
        int64_t mid = (lo + hi) >> 1;
        if (offsets[mid + 1] <= row) lo = mid + 1; else hi = mid;
    }
    return lo;
}

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

// sums[s] += sum of x (mean == null) or of (x - mean_s)^2 over the block's rows.
// A block that lies inside one sample reduces in shared memory and issues one
// atomic; the few blocks that straddle a boundary add per thread.
template <typename T>
__global__ void ln_sum_kernel(const T *__restrict__ x, const int64_t *__restrict__ offsets,
                              const float *__restrict__ mean, float *sums, int64_t N, int64_t S, int C) {
    __shared__ float scratch[LN_THREADS / 32];
    const int64_t row0 = (int64_t)blockIdx.x * LN_ROWS, row1 = min(N, row0 + LN_ROWS);
    const int64_t s_first = sample_of(offsets, S, row0), s_last = sample_of(offsets, S, row1 - 1);
    const int64_t e0 = row0 * C, e1 = row1 * C;
    if (s_first == s_last) {
        const float mu = mean ? mean[s_first] : 0.f;
        float v = 0.f;
        for (int64_t e = e0 + threadIdx.x; e < e1; e += LN_THREADS) {
            const float d = to_f32<T>(x[e]) - mu;
            v += mean ? d * d : d;
        }
        v = block_sum(v, scratch);
        if (threadIdx.x == 0) atomicAdd(sums + s_first, v);
        return;
    }
    for (int64_t r = row0 + threadIdx.x / 32; r < row1; r += LN_THREADS / 32) {
        const int64_t s = sample_of(offsets, S, r);
        const float mu = mean ? mean[s] : 0.f;
        float v = 0.f;
        for (int c = threadIdx.x & 31; c < C; c += 32) {
            const float d = to_f32<T>(x[r * C + c]) - mu;
            v += mean ? d * d : d;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        if ((threadIdx.x & 31) == 0) atomicAdd(sums + s, v);
    }
}

// pass 1 -> mean; pass 2 -> rstd
__global__ void ln_stats_kernel(const float *__restrict__ sums, const int64_t *__restrict__ offsets, float *mean,
                                float *rstd, int64_t S, int C, float eps, int second) {
    int64_t s = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (s >= S) return;
    const int64_t len = offsets[s + 1] - offsets[s];
    const float n = (float)(len > 0 ? len : 1) * (float)C;
    if (!second) mean[s] = sums[s] / n;
    else rstd[s] = 1.f / sqrtf(sums[s] / n + eps);
}

template <typename T>
__global__ void ln_apply_kernel(const T *__restrict__ x, const int64_t *__restrict__ offsets,
                                const float *__restrict__ mean, const float *__restrict__ rstd,
                                const float *__restrict__ weight, const float *__restrict__ bias,
                                const T *__restrict__ residual, T *y, int64_t N, int64_t S, int C, int relu) {
    const int64_t row0 = (int64_t)blockIdx.x * LN_ROWS, row1 = min(N, row0 + LN_ROWS);
    for (int64_t r = row0 + threadIdx.x / 32; r < row1; r += LN_THREADS / 32) {
        const int64_t s = sample_of(offsets, S, r);
        const float mu = mean[s], rs = rstd[s];
        for (int c = threadIdx.x & 31; c < C; c += 32) {
            float v = (to_f32<T>(x[r * C + c]) - mu) * rs;
            if (weight) v = v * weight[c] + bias[c];
            if (residual) v += to_f32<T>(residual[r * C + c]);
            if (relu) v = fmaxf(v, 0.f);
            y[r * C + c] = from_f32<T>(v);
        }
    }
}

// Per-sample sums of gh and gh * xh, per-channel sums of g' * xh and g', and
// (optionally) the masked gradient for the residual branch.  Partial sums stay in
// registers while a thread's rows belong to one sample; a block inside one sample
// reduces in shared memory and issues one atomic per sum, and one per channel.
template <typename T>
__global__ void ln_bwd_sums_kernel(const T *__restrict__ g, const T *__restrict__ x, const T *__restrict__ y,
                                   const int64_t *__restrict__ offsets, const float *__restrict__ mean,
                                   const float *__restrict__ rstd, const float *__restrict__ weight, float *s1,
                                   float *s2, float *dweight, float *dbias, T *dresidual, int64_t N, int64_t S,
                                   int C, int relu) {
    __shared__ float scratch[LN_THREADS / 32];
    __shared__ float col_w[LN_THREADS / 32][32], col_b[LN_THREADS / 32][32];
    const int64_t row0 = (int64_t)blockIdx.x * LN_ROWS, row1 = min(N, row0 + LN_ROWS);
    const int lane = threadIdx.x & 31, rl = threadIdx.x / 32;
    const int64_t s_first = sample_of(offsets, S, row0), s_last = sample_of(offsets, S, row1 - 1);
    const bool uniform = s_first == s_last;
    float a = 0.f, b = 0.f;     // running sums of gh and gh * xh for sample `cur`
    int64_t cur = s_first;
    for (int c0 = 0; c0 < C; c0 += 32) {
        const int c = c0 + lane;
        const float w = (weight && c < C) ? weight[c] : 1.f;
        float dw = 0.f, db = 0.f;
        for (int64_t r = row0 + rl; r < row1; r += LN_THREADS / 32) {
            const int64_t s = uniform ? s_first : sample_of(offsets, S, r);
            if (s != cur) {
                atomicAdd(s1 + cur, a);
                atomicAdd(s2 + cur, b);
                a = b = 0.f;
                cur = s;
            }
            if (c < C) {
                float gv = to_f32<T>(g[r * C + c]);
                if (relu && !(to_f32<T>(y[r * C + c]) > 0.f)) gv = 0.f;
                if (dresidual) dresidual[r * C + c] = from_f32<T>(gv);
                const float xh = (to_f32<T>(x[r * C + c]) - mean[s]) * rstd[s];
                a += gv * w;
                b += gv * w * xh;
                dw += gv * xh;
                db += gv;
            }
        }
        if (dweight) {
            col_w[rl][lane] = dw;
            col_b[rl][lane] = db;
            __syncthreads();
            if (rl == 0 && c < C) {
                float tw = 0.f, tb = 0.f;
                for (int q = 0; q < LN_THREADS / 32; ++q) tw += col_w[q][lane], tb += col_b[q][lane];
                atomicAdd(dweight + c, tw);
                atomicAdd(dbias + c, tb);
            }
            __syncthreads();
        }
    }
    if (uniform) {
        a = block_sum(a, scratch);
        b = block_sum(b, scratch);
        if (threadIdx.x == 0) {
            atomicAdd(s1 + s_first, a);
            atomicAdd(s2 + s_first, b);
        }
    } else {
        atomicAdd(s1 + cur, a);
        atomicAdd(s2 + cur, b);
    }
}

template <typename T>
__global__ void ln_bwd_apply_kernel(const T *__restrict__ g, const T *__restrict__ x, const T *__restrict__ y,
                                    const int64_t *__restrict__ offsets, const float *__restrict__ mean,
                                    const float *__restrict__ rstd, const float *__restrict__ weight,
                                    const float *__restrict__ s1, const float *__restrict__ s2, T *dx, int64_t N,
                                    int64_t S, int C, int relu) {
    const int64_t row0 = (int64_t)blockIdx.x * LN_ROWS, row1 = min(N, row0 + LN_ROWS);
    for (int64_t r = row0 + threadIdx.x / 32; r < row1; r += LN_THREADS / 32) {
        const int64_t s = sample_of(offsets, S, r);
        const float mu = mean[s], rs = rstd[s];
        const float inv_n = 1.f / ((float)(offsets[s + 1] - offsets[s]) * (float)C);
        const float m1 = s1[s] * inv_n, m2 = s2[s] * inv_n;
        for (int c = threadIdx.x & 31; c < C; c += 32) {
            float gv = to_f32<T>(g[r * C + c]);
            if (relu && !(to_f32<T>(y[r * C + c]) > 0.f)) gv = 0.f;
            const float gh = weight ? gv * weight[c] : gv;
            const float xh = (to_f32<T>(x[r * C + c]) - mu) * rs;
            dx[r * C + c] = from_f32<T>(rs * (gh - m1 - xh * m2));
        }
    }
}

struct LnWs {
    int64_t *offsets;
    float *sums;   // 2 * S
    void *cub_tmp;
    size_t cub_bytes;
};

size_t carve_ln(void *ws, int64_t S, LnWs *out) {
    Carver c(ws);
    LnWs w;
    w.offsets = c.take<int64_t>((size_t)S + 1);
    w.sums = c.take<float>((size_t)2 * S + 1);
    size_t bytes = 0;
    cub::DeviceScan::ExclusiveSum(nullptr, bytes, (const int64_t *)nullptr, (int64_t *)nullptr, (int)std::max<int64_t>(S, 1));
    w.cub_bytes = bytes;
    w.cub_tmp = c.take<char>(bytes);
    if (out) *out = w;
    return c.off;
}

int ln_offsets(const int64_t *d_lengths, int64_t S, int64_t N, const LnWs &w, cudaStream_t stream) {
    size_t bytes = w.cub_bytes;
    PCX_CUDA(cub::DeviceScan::ExclusiveSum(w.cub_tmp, bytes, d_lengths, w.offsets, (int)S, stream));
    ln_tail_kernel<<<1, 32, 0, stream>>>(w.offsets, S, N);
    PCX_LAUNCH_CHECK();
    return PCX_OK;
}

bool ln_sizes_ok(int64_t N, int64_t S, int C, int dtype) {
    return N >= 0 && S > 0 && S <= INT32_MAX && C > 0 && (dtype == PCX_F32 || dtype == PCX_F16 || dtype == PCX_BF16);
}

#define PCX_LN_BY_DTYPE(dtype, CALL)                              \
    do {                                                          \
        if ((dtype) == PCX_F32) { using T = float; CALL; }        \
        else if ((dtype) == PCX_F16) { using T = __half; CALL; }  \
        else { using T = __nv_bfloat16; CALL; }                   \
    } while (0)

}  // namespace
}  // namespace pcx

using namespace pcx;

extern "C" {

size_t pcx_ragged_layer_norm_workspace_bytes(int64_t S) { return S <= 0 ? 0 : carve_ln(nullptr, S, nullptr); }

int pcx_ragged_layer_norm(const void *d_x, const int64_t *d_lengths, const float *d_weight, const float *d_bias,
                          const void *d_residual, void *d_y, float *d_mean, float *d_rstd, int64_t N, int64_t S, int C,
                          double eps, int relu, int dtype, void *d_ws, size_t ws_bytes, void *stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    if (!ln_sizes_ok(N, S, C, dtype)) PCX_FAIL(PCX_E_ARG, "pcx_ragged_layer_norm: bad sizes or dtype");
    if (!d_lengths || !d_mean || !d_rstd || !d_ws || (N > 0 && (!d_x || !d_y)) || ((d_weight == nullptr) != (d_bias == nullptr)))
        PCX_FAIL(PCX_E_ARG, "pcx_ragged_layer_norm: null pointer (weight and bias come together)");
    if ((uintptr_t)d_ws % 256) PCX_FAIL(PCX_E_ALIGN, "pcx_ragged_layer_norm: workspace must be 256-byte aligned");
    LnWs w;
    size_t need = carve_ln(d_ws, S, &w);
    if (ws_bytes < need) PCX_FAIL(PCX_E_CAPACITY, "pcx_ragged_layer_norm: workspace %zu < %zu bytes", ws_bytes, need);
    if (int rc = ln_offsets(d_lengths, S, N, w, stream)) return rc;
    PCX_CUDA(cudaMemsetAsync(w.sums, 0, (size_t)2 * S * sizeof(float), stream));
    const unsigned grid = (unsigned)((N + LN_ROWS - 1) / LN_ROWS), sgrid = (unsigned)((S + 127) / 128);
    if (N > 0) {
        PCX_LN_BY_DTYPE(dtype, (ln_sum_kernel<T><<<grid, LN_THREADS, 0, stream>>>((const T *)d_x, w.offsets, nullptr, w.sums, N, S, C)));
        PCX_LAUNCH_CHECK();
    }
    ln_stats_kernel<<<sgrid, 128, 0, stream>>>(w.sums, w.offsets, d_mean, d_rstd, S, C, (float)eps, 0);
    PCX_LAUNCH_CHECK();
    if (N > 0) {
        PCX_LN_BY_DTYPE(dtype, (ln_sum_kernel<T><<<grid, LN_THREADS, 0, stream>>>((const T *)d_x, w.offsets, d_mean, w.sums + S, N, S, C)));
        PCX_LAUNCH_CHECK();
    }
    ln_stats_kernel<<<sgrid, 128, 0, stream>>>(w.sums + S, w.offsets, d_mean, d_rstd, S, C, (float)eps, 1);
    PCX_LAUNCH_CHECK();
    if (N > 0) {
        prof_begin("ln_apply_kernel", stream);
        PCX_LN_BY_DTYPE(dtype, (ln_apply_kernel<T><<<grid, LN_THREADS, 0, stream>>>(
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
    PCX_LN_BY_DTYPE(dtype, (ln_bwd_sums_kernel<T><<<grid, LN_THREADS, 0, stream>>>(
                               (const T *)d_grad_y, (const T *)d_x, (const T *)d_y, w.offsets, d_mean, d_rstd, d_weight,
                               w.sums, w.sums + S, d_grad_weight, d_grad_bias, (T *)d_grad_residual, N, S, C, relu)));
    PCX_LAUNCH_CHECK();
    PCX_LN_BY_DTYPE(dtype, (ln_bwd_apply_kernel<T><<<grid, LN_THREADS, 0, stream>>>(
                               (const T *)d_grad_y, (const T *)d_x, (const T *)d_y, w.offsets, d_mean, d_rstd, d_weight,
                               w.sums, w.sums + S, (T *)d_grad_x, N, S, C, relu)));
    PCX_LAUNCH_CHECK();
    return PCX_OK;
}

}  // extern "C"
