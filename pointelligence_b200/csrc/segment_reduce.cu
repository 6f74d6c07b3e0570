// Segment reductions of the backbone step: per-sample statistics and global
// pooling over contiguous row segments, and max / mean pooling over neighbour
// lists.  HBM-bound byte work: rows are read once, coalesced along channels,
// accumulated in fp32 registers and rounded once.
//
//   segment_reduce          out[s] = reduce_{n in segment s} x[n]
//                           (sparse_engines/large_segment_reduce_triton.py:25-77 of the reference)
//   segment_reduce_backward (large_segment_reduce_triton.py:94-166)
//   indexed_segment_reduce  y[k]   = reduce_{e in list k} x[indices[e]]
//                           (sparse_engines/indexed_segment_reduce_triton.py:25-63)
//   indexed_segment_reduce_backward (indexed_segment_reduce_triton.py:84-140)
//
// Conventions kept from the reference: op 0 sum, 1 mean, 2 max, 3 min; an empty
// contiguous segment gives 0 for sum and mean (division by max(len, 1)) and
// -inf / +inf for max / min; an empty neighbour list gives 0 (sum), NaN (mean,
// 0/0) and -inf / +inf; max / min gradients go to every element that equals the
// reduced value; fp16 results of the contiguous reduction are clamped to +-65504.
#include <cub/cub.cuh>

#include "rowwise.cuh"
#include "sparse_kernels.cuh"

namespace pcx {
namespace {

enum { OP_SUM = 0, OP_MEAN = 1, OP_MAX = 2, OP_MIN = 3 };

__device__ __forceinline__ float neutral_of(int op) {
    return op == OP_MAX ? -INFINITY : op == OP_MIN ? INFINITY : 0.f;
}
__device__ __forceinline__ float combine(float a, float b, int op) {
    return op == OP_MAX ? fmaxf(a, b) : op == OP_MIN ? fminf(a, b) : a + b;
}
// float max / min through the integer atomics (the sign decides which ordering applies)
__device__ __forceinline__ void atomic_combine(float *addr, float v, int op) {
    if (op == OP_MAX) {
        if (!signbit(v)) atomicMax(reinterpret_cast<int *>(addr), __float_as_int(v));
        else atomicMin(reinterpret_cast<unsigned int *>(addr), __float_as_uint(v));
    } else if (op == OP_MIN) {
        if (!signbit(v)) atomicMin(reinterpret_cast<int *>(addr), __float_as_int(v));
        else atomicMax(reinterpret_cast<unsigned int *>(addr), __float_as_uint(v));
    } else {
        atomicAdd(addr, v);
    }
}

__global__ void set_tail_kernel(int64_t *offsets, int64_t S, int64_t total) {
    if (threadIdx.x == 0 && blockIdx.x == 0) {
        offsets[S] = total;
        if (S == 0) offsets[0] = 0;
    }
}

__global__ void fill_kernel(float *p, int64_t n, float v) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) p[i] = v;
}

// A block owns SEG_ROWS consecutive rows; a thread keeps one vector column (VN channels,
// one 16-byte access when VN > 1) and walks the rows of its row lane.  A block inside one
// segment folds its row lanes in shared memory and issues one atomic per channel; blocks
// that straddle a boundary flush per thread whenever the segment changes.
constexpr int SEG_ROWS = 1024;
constexpr int SEG_THREADS = 256;

template <typename T, int VN>
__global__ void seg_reduce_kernel(const T *__restrict__ x, const int64_t *__restrict__ offsets, float *acc,
                                  int64_t N, int64_t S, int C, int op) {
    __shared__ float fold[SEG_THREADS * VN];
    const int64_t row0 = (int64_t)blockIdx.x * SEG_ROWS, row1 = min(N, row0 + SEG_ROWS);
    const int64_t s_first = segment_of_row(offsets, S, row0);
    const bool uniform = s_first == segment_of_row(offsets, S, row1 - 1);
    const RowLayout L(C, VN);
    for (int cp = 0; cp * L.vcb < L.vc_total; ++cp) {
        const int vcol = cp * L.vcb + L.vc;
        const bool active = vcol < L.vc_total && L.lane < L.lanes;
        float v[VN];
#pragma unroll
        for (int i = 0; i < VN; ++i) v[i] = neutral_of(op);
        int64_t cur = s_first;
        if (active) {
#pragma unroll 4
            for (int64_t r = row0 + L.lane; r < row1; r += L.lanes) {
                const int64_t s = uniform ? s_first : segment_of_row(offsets, S, r);
                if (s != cur) {
#pragma unroll
                    for (int i = 0; i < VN; ++i) {
                        atomic_combine(acc + cur * C + vcol * VN + i, v[i], op);
                        v[i] = neutral_of(op);
                    }
                    cur = s;
                }
                float in[VN];
                load_vec<T, VN>(x + r * C + (int64_t)vcol * VN, in);
#pragma unroll
                for (int i = 0; i < VN; ++i) v[i] = combine(v[i], in[i], op);
            }
        }
        if (uniform) {
#pragma unroll
            for (int i = 0; i < VN; ++i) fold[(L.lane * L.vcb + L.vc) * VN + i] = v[i];
            __syncthreads();
            const int cols = L.vcb * VN;
            for (int t = threadIdx.x; t < cols; t += SEG_THREADS) {
                const int c = cp * cols + t;
                if (c < C) {
                    float f = neutral_of(op);
                    for (int q = 0; q < L.lanes; ++q) f = combine(f, fold[q * cols + t], op);
                    atomic_combine(acc + s_first * C + c, f, op);
                }
            }
            __syncthreads();
        } else if (active) {
#pragma unroll
            for (int i = 0; i < VN; ++i) atomic_combine(acc + cur * C + vcol * VN + i, v[i], op);
        }
    }
}

template <typename T>
__global__ void seg_finalize_kernel(const float *__restrict__ acc, const int64_t *__restrict__ offsets, T *out,
                                    int64_t S, int C, int op, int clamp_fp16) {
    int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= S * C) return;
    float v = acc[e];
    if (op == OP_MEAN) {
        int64_t s = e / C, len = offsets[s + 1] - offsets[s];
        v = v / (float)(len > 0 ? len : 1);
    }
    if (clamp_fp16) v = fminf(fmaxf(v, -65504.f), 65504.f);
    out[e] = from_f32<T>(v);
}

template <typename T, int VN>
__global__ void seg_reduce_bwd_kernel(const T *__restrict__ gout, const T *__restrict__ x, const T *__restrict__ outv,
                                      const int64_t *__restrict__ offsets, T *gin, int64_t N, int64_t S, int C,
                                      int op) {
    const int64_t row0 = (int64_t)blockIdx.x * SEG_ROWS, row1 = min(N, row0 + SEG_ROWS);
    const int64_t s_first = segment_of_row(offsets, S, row0);
    const bool uniform = s_first == segment_of_row(offsets, S, row1 - 1);
    const RowLayout L(C, VN);
    for (int cp = 0; cp * L.vcb < L.vc_total; ++cp) {
        const int vcol = cp * L.vcb + L.vc;
        if (vcol >= L.vc_total || L.lane >= L.lanes) continue;
#pragma unroll 2
        for (int64_t r = row0 + L.lane; r < row1; r += L.lanes) {
            const int64_t s = uniform ? s_first : segment_of_row(offsets, S, r);
            const float inv = op == OP_MEAN ? 1.f / (float)max((int64_t)1, offsets[s + 1] - offsets[s]) : 1.f;
            float gv[VN], xv[VN], ov[VN];
            load_vec<T, VN>(gout + s * C + (int64_t)vcol * VN, gv);
            if (op >= OP_MAX) {
                load_vec<T, VN>(x + r * C + (int64_t)vcol * VN, xv);
                load_vec<T, VN>(outv + s * C + (int64_t)vcol * VN, ov);
            }
#pragma unroll
            for (int i = 0; i < VN; ++i) {
                gv[i] *= inv;
                if (op >= OP_MAX && !(xv[i] == ov[i])) gv[i] = 0.f;
            }
            store_vec<T, VN>(gin + r * C + (int64_t)vcol * VN, gv);
        }
    }
}

// Output rows side by side in a block: a thread keeps one vector column of one output row
// and walks that row's list (C = 64 bf16: 8 threads per output row, 32 rows per block).
constexpr int IDX_THREADS = 256;

template <typename T, int VN>
__global__ void idx_reduce_kernel(const T *__restrict__ x, const int32_t *__restrict__ indices,
                                  const int64_t *__restrict__ offsets, T *y, int64_t K, int C, int op) {
    const RowLayout L(C, VN);
    const int64_t k = (int64_t)blockIdx.x * L.lanes + L.lane;
    if (L.lane >= L.lanes || k >= K) return;
    const int64_t lo = offsets[k], hi = offsets[k + 1];
    for (int cp = 0; cp * L.vcb < L.vc_total; ++cp) {
        const int vcol = cp * L.vcb + L.vc;
        if (vcol >= L.vc_total) continue;
        float v[VN];
#pragma unroll
        for (int i = 0; i < VN; ++i) v[i] = neutral_of(op);
#pragma unroll 4
        for (int64_t e = lo; e < hi; ++e) {
            float in[VN];
            load_vec<T, VN>(x + (int64_t)indices[e] * C + (int64_t)vcol * VN, in);
#pragma unroll
            for (int i = 0; i < VN; ++i) v[i] = combine(v[i], in[i], op);
        }
        if (op == OP_MEAN) {
#pragma unroll
            for (int i = 0; i < VN; ++i) v[i] = v[i] / (float)(hi - lo);
        }
        store_vec<T, VN>(y + k * C + (int64_t)vcol * VN, v);
    }
}

template <typename T, int VN>
__global__ void idx_reduce_bwd_kernel(const T *__restrict__ gy, const T *__restrict__ x, const T *__restrict__ y,
                                      const int32_t *__restrict__ indices, const int64_t *__restrict__ offsets,
                                      float *acc, int64_t K, int C, int op) {
    const RowLayout L(C, VN);
    const int64_t k = (int64_t)blockIdx.x * L.lanes + L.lane;
    if (L.lane >= L.lanes || k >= K) return;
    const int64_t lo = offsets[k], hi = offsets[k + 1];
    for (int cp = 0; cp * L.vcb < L.vc_total; ++cp) {
        const int vcol = cp * L.vcb + L.vc;
        if (vcol >= L.vc_total) continue;
        float g[VN], target[VN];
        load_vec<T, VN>(gy + k * C + (int64_t)vcol * VN, g);
        if (op >= OP_MAX) load_vec<T, VN>(y + k * C + (int64_t)vcol * VN, target);
        if (op == OP_MEAN) {
#pragma unroll
            for (int i = 0; i < VN; ++i) g[i] = g[i] / (float)(hi - lo);
        }
        for (int64_t e = lo; e < hi; ++e) {
            const int64_t at = (int64_t)indices[e] * C + (int64_t)vcol * VN;
            float add[VN];
#pragma unroll
            for (int i = 0; i < VN; ++i) add[i] = g[i];
            if (op >= OP_MAX) {
                float in[VN];
                load_vec<T, VN>(x + at, in);
#pragma unroll
                for (int i = 0; i < VN; ++i)
                    if (!(in[i] == target[i])) add[i] = 0.f;
            }
            if constexpr (VN % 4 == 0) {
#pragma unroll
                for (int i = 0; i < VN; i += 4)
                    atomicAdd(reinterpret_cast<float4 *>(acc + at + i), make_float4(add[i], add[i + 1], add[i + 2], add[i + 3]));
            } else {
#pragma unroll
                for (int i = 0; i < VN; ++i)
                    if (add[i] != 0.f || op < OP_MAX) atomicAdd(acc + at + i, add[i]);
            }
        }
    }
}

static inline unsigned idx_grid(int64_t K, int C, int vn) {
    const int vc_total = C / vn;
    const int vcb = vc_total < IDX_THREADS ? vc_total : IDX_THREADS;
    const int lanes = IDX_THREADS / vcb;
    return (unsigned)((K + lanes - 1) / lanes);
}

struct OffsWs {
    int64_t *offsets;
    float *acc;
    void *cub_tmp;
    size_t cub_bytes;
};

size_t carve_offsets(void *ws, int64_t S, size_t acc_elems, OffsWs *out) {
    Carver c(ws);
    OffsWs w;
    w.offsets = c.take<int64_t>((size_t)S + 1);
    w.acc = c.take<float>(acc_elems ? acc_elems : 1);
    size_t bytes = 0;
    cub::DeviceScan::ExclusiveSum(nullptr, bytes, (const int64_t *)nullptr, (int64_t *)nullptr, (int)std::max<int64_t>(S, 1));
    w.cub_bytes = bytes;
    w.cub_tmp = c.take<char>(bytes);
    if (out) *out = w;
    return c.off;
}

int scan_lengths(const int64_t *d_lengths, int64_t S, int64_t total, const OffsWs &w, cudaStream_t stream) {
    if (S > 0) {
        size_t bytes = w.cub_bytes;
        PCX_CUDA(cub::DeviceScan::ExclusiveSum(w.cub_tmp, bytes, d_lengths, w.offsets, (int)S, stream));
    }
    set_tail_kernel<<<1, 32, 0, stream>>>(w.offsets, S, total);
    PCX_LAUNCH_CHECK();
    return PCX_OK;
}

bool sizes_ok(int64_t rows, int64_t S, int C, int op, int dtype) {
    return rows >= 0 && S >= 0 && S <= INT32_MAX && C > 0 && op >= 0 && op <= 3 &&
           (dtype == PCX_F32 || dtype == PCX_F16 || dtype == PCX_BF16);
}

// CALL sees T and VN (channels per access: 16 bytes' worth when `vec`, else 1)
#define PCX_BY_DTYPE_VEC(dtype, vec, CALL)                                                                       \
    do {                                                                                                         \
        if ((dtype) == PCX_F32) { using T = float; if (vec) { constexpr int VN = 4; CALL; } else { constexpr int VN = 1; CALL; } }       \
        else if ((dtype) == PCX_F16) { using T = __half; if (vec) { constexpr int VN = 8; CALL; } else { constexpr int VN = 1; CALL; } }  \
        else { using T = __nv_bfloat16; if (vec) { constexpr int VN = 8; CALL; } else { constexpr int VN = 1; CALL; } }                   \
    } while (0)

#define PCX_BY_DTYPE(dtype, CALL)                    \
    do {                                             \
        if ((dtype) == PCX_F32) { using T = float; CALL; }             \
        else if ((dtype) == PCX_F16) { using T = __half; CALL; }       \
        else { using T = __nv_bfloat16; CALL; }                        \
    } while (0)

}  // namespace
}  // namespace pcx

using namespace pcx;

extern "C" {

size_t pcx_segment_reduce_workspace_bytes(int64_t S, int C) {
    if (S < 0 || C <= 0) return 0;
    return carve_offsets(nullptr, S, (size_t)S * C, nullptr);
}

int pcx_segment_reduce(const void *d_x, const int64_t *d_lengths, void *d_out, int64_t N, int64_t S, int C, int op,
                       int dtype, void *d_ws, size_t ws_bytes, void *stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    if (!sizes_ok(N, S, C, op, dtype)) PCX_FAIL(PCX_E_ARG, "pcx_segment_reduce: bad sizes, op or dtype");
    if (S == 0) return PCX_OK;
    if (!d_lengths || !d_out || !d_ws || (N > 0 && !d_x)) PCX_FAIL(PCX_E_ARG, "pcx_segment_reduce: null pointer");
    if ((uintptr_t)d_ws % 256) PCX_FAIL(PCX_E_ALIGN, "pcx_segment_reduce: workspace must be 256-byte aligned");
    OffsWs w;
    size_t need = carve_offsets(d_ws, S, (size_t)S * C, &w);
    if (ws_bytes < need) PCX_FAIL(PCX_E_CAPACITY, "pcx_segment_reduce: workspace %zu < %zu bytes", ws_bytes, need);
    if (int rc = scan_lengths(d_lengths, S, N, w, stream)) return rc;
    const int64_t elems = S * C;
    const float init = op == OP_MAX ? -INFINITY : op == OP_MIN ? INFINITY : 0.f;
    fill_kernel<<<(unsigned)((elems + 255) / 256), 256, 0, stream>>>(w.acc, elems, init);
    PCX_LAUNCH_CHECK();
    if (N > 0) {
        const unsigned grid = (unsigned)((N + SEG_ROWS - 1) / SEG_ROWS);
        const bool vec = vec_ok(C, dtype, {d_x});
        prof_begin("seg_reduce_kernel", stream);
        PCX_BY_DTYPE_VEC(dtype, vec, (seg_reduce_kernel<T, VN><<<grid, SEG_THREADS, 0, stream>>>((const T *)d_x, w.offsets, w.acc, N, S, C, op)));
        prof_end(stream);
        PCX_LAUNCH_CHECK();
    }
    PCX_BY_DTYPE(dtype, (seg_finalize_kernel<T><<<(unsigned)((elems + 255) / 256), 256, 0, stream>>>(
                            w.acc, w.offsets, (T *)d_out, S, C, op, dtype == PCX_F16)));
    PCX_LAUNCH_CHECK();
    return PCX_OK;
}

int pcx_segment_reduce_backward(const void *d_grad_out, const void *d_x, const void *d_out, const int64_t *d_lengths,
                                void *d_grad_x, int64_t N, int64_t S, int C, int op, int dtype, void *d_ws,
                                size_t ws_bytes, void *stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    if (!sizes_ok(N, S, C, op, dtype)) PCX_FAIL(PCX_E_ARG, "pcx_segment_reduce_backward: bad sizes, op or dtype");
    if (N == 0) return PCX_OK;
    if (!d_grad_out || !d_lengths || !d_grad_x || !d_ws || (op >= OP_MAX && (!d_x || !d_out)))
        PCX_FAIL(PCX_E_ARG, "pcx_segment_reduce_backward: null pointer");
    if ((uintptr_t)d_ws % 256) PCX_FAIL(PCX_E_ALIGN, "pcx_segment_reduce_backward: workspace must be 256-byte aligned");
    OffsWs w;
    size_t need = carve_offsets(d_ws, S, 0, &w);
    if (ws_bytes < need) PCX_FAIL(PCX_E_CAPACITY, "pcx_segment_reduce_backward: workspace %zu < %zu bytes", ws_bytes, need);
    if (int rc = scan_lengths(d_lengths, S, N, w, stream)) return rc;
    const unsigned grid = (unsigned)((N + SEG_ROWS - 1) / SEG_ROWS);
    const bool vec = vec_ok(C, dtype, {d_grad_out, op >= OP_MAX ? d_x : nullptr, op >= OP_MAX ? d_out : nullptr, d_grad_x});
    PCX_BY_DTYPE_VEC(dtype, vec, (seg_reduce_bwd_kernel<T, VN><<<grid, SEG_THREADS, 0, stream>>>(
                                     (const T *)d_grad_out, (const T *)d_x, (const T *)d_out, w.offsets, (T *)d_grad_x,
                                     N, S, C, op)));
    PCX_LAUNCH_CHECK();
    return PCX_OK;
}

size_t pcx_indexed_segment_reduce_workspace_bytes(int64_t K, int64_t n_x, int C, int dtype, int backward) {
    if (K < 0 || n_x < 0 || C <= 0) return 0;
    return carve_offsets(nullptr, K, backward && dtype != PCX_F32 ? (size_t)n_x * C : 0, nullptr);
}

int pcx_indexed_segment_reduce(const void *d_x, const int32_t *d_indices, const int64_t *d_lengths, void *d_y,
                               int64_t n_x, int64_t E, int64_t K, int C, int op, int dtype, void *d_ws, size_t ws_bytes,
                               void *stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    if (!sizes_ok(E, K, C, op, dtype) || n_x < 0) PCX_FAIL(PCX_E_ARG, "pcx_indexed_segment_reduce: bad sizes, op or dtype");
    if (K == 0) return PCX_OK;
    if (!d_lengths || !d_y || !d_ws || (E > 0 && (!d_x || !d_indices)))
        PCX_FAIL(PCX_E_ARG, "pcx_indexed_segment_reduce: null pointer");
    if ((uintptr_t)d_ws % 256) PCX_FAIL(PCX_E_ALIGN, "pcx_indexed_segment_reduce: workspace must be 256-byte aligned");
    OffsWs w;
    size_t need = carve_offsets(d_ws, K, 0, &w);
    if (ws_bytes < need) PCX_FAIL(PCX_E_CAPACITY, "pcx_indexed_segment_reduce: workspace %zu < %zu bytes", ws_bytes, need);
    if (int rc = scan_lengths(d_lengths, K, E, w, stream)) return rc;
    const bool vec = vec_ok(C, dtype, {d_x, d_y});
    prof_begin("idx_reduce_kernel", stream);
    PCX_BY_DTYPE_VEC(dtype, vec, (idx_reduce_kernel<T, VN><<<idx_grid(K, C, VN), IDX_THREADS, 0, stream>>>(
                                     (const T *)d_x, d_indices, w.offsets, (T *)d_y, K, C, op)));
    prof_end(stream);
    PCX_LAUNCH_CHECK();
    return PCX_OK;
}

int pcx_indexed_segment_reduce_backward(const void *d_grad_y, const void *d_x, const void *d_y,
                                        const int32_t *d_indices, const int64_t *d_lengths, void *d_grad_x,
                                        int64_t n_x, int64_t E, int64_t K, int C, int op, int dtype, void *d_ws,
                                        size_t ws_bytes, void *stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    if (!sizes_ok(E, K, C, op, dtype) || n_x < 0)
        PCX_FAIL(PCX_E_ARG, "pcx_indexed_segment_reduce_backward: bad sizes, op or dtype");
    if (n_x == 0) return PCX_OK;
    if (!d_grad_x || !d_ws || (K > 0 && (!d_grad_y || !d_lengths)) || (E > 0 && !d_indices) ||
        (op >= OP_MAX && E > 0 && (!d_x || !d_y)))
        PCX_FAIL(PCX_E_ARG, "pcx_indexed_segment_reduce_backward: null pointer");
    if ((uintptr_t)d_ws % 256) PCX_FAIL(PCX_E_ALIGN, "pcx_indexed_segment_reduce_backward: workspace must be 256-byte aligned");
    OffsWs w;
    const size_t acc_elems = dtype != PCX_F32 ? (size_t)n_x * C : 0;
    size_t need = carve_offsets(d_ws, K, acc_elems, &w);
    if (ws_bytes < need)
        PCX_FAIL(PCX_E_CAPACITY, "pcx_indexed_segment_reduce_backward: workspace %zu < %zu bytes", ws_bytes, need);
    if (int rc = scan_lengths(d_lengths, K, E, w, stream)) return rc;
    float *acc = dtype == PCX_F32 ? (float *)d_grad_x : w.acc;
    PCX_CUDA(cudaMemsetAsync(acc, 0, (size_t)n_x * C * sizeof(float), stream));
    if (K > 0 && E > 0) {
        const bool vec = vec_ok(C, dtype, {d_grad_y, op >= OP_MAX ? d_x : nullptr, op >= OP_MAX ? d_y : nullptr, acc});
        PCX_BY_DTYPE_VEC(dtype, vec, (idx_reduce_bwd_kernel<T, VN><<<idx_grid(K, C, VN), IDX_THREADS, 0, stream>>>(
                                         (const T *)d_grad_y, (const T *)d_x, (const T *)d_y, d_indices, w.offsets, acc,
                                         K, C, op)));
        PCX_LAUNCH_CHECK();
    }
    if (dtype != PCX_F32) return round_accumulator(acc, d_grad_x, n_x * C, dtype, stream);
    return PCX_OK;
}

}  // extern "C"
