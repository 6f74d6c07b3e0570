// CUDA-core engines for MVMR and VVOR: any element type, any channel counts,
// any number of groups, IEEE fp32 multiply-add.  They serve the shapes the
// tensor-core engine does not take (fp32 operands, channel counts that are not
// multiples of 16, grouped weights, triplets that are not sorted by tap) and
// are the arithmetic reference for it in the GPU tests.
//
// Sorted triplets are cut into chunks of one tap so that the weight tile is
// staged in shared memory once per chunk and every thread keeps a 4x4 block of
// accumulators in registers; the partial sums go to an fp32 accumulator with
// red.global.add.f32 and are rounded once into the output element type.
#include "sparse_kernels.cuh"

namespace pcx {

// cum[k] = number of L-triplet chunks in the taps before k (one block, any K)
__global__ void chunk_table_kernel(const int64_t *__restrict__ seg, int K, int L, int32_t *cum) {
    __shared__ int32_t warp_sums[32];
    __shared__ int32_t carry;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
    if (tid == 0) carry = 0;
    __syncthreads();
    for (int base = 0; base < K; base += blockDim.x) {
        int k = base + tid;
        int32_t v = k < K ? (int32_t)((seg[k + 1] - seg[k] + L - 1) / L) : 0;
        int32_t inc = v;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            int32_t n = __shfl_up_sync(0xffffffffu, inc, o);
            if (lane >= o) inc += n;
        }
        if (lane == 31) warp_sums[warp] = inc;
        __syncthreads();
        int32_t before = carry;
        for (int w = 0; w < warp; ++w) before += warp_sums[w];
        if (k < K) cum[k] = before + inc - v;
        __syncthreads();
        if (tid == 0) {
            int32_t t = carry;
            for (int w = 0; w < nwarps; ++w) t += warp_sums[w];
            carry = t;
        }
        __syncthreads();
    }
    if (tid == 0) cum[K] = carry;
}

namespace {

// chunk id -> (tap, first triplet, rows); false when the id is past the end
__device__ __forceinline__ bool locate_chunk(const int32_t *__restrict__ cum, const int64_t *__restrict__ seg,
                                             int K, int L, int chunk, int *tap, int64_t *t0, int *rows) {
    if (chunk >= cum[K]) return false;
    int lo = 0, hi = K;  // largest k with cum[k] <= chunk
    while (hi - lo > 1) {
        int mid = (lo + hi) >> 1;
        if (cum[mid] <= chunk) lo = mid; else hi = mid;
    }
    // skip empty taps that share the same cumulative value
    while (lo + 1 < K && cum[lo + 1] <= chunk) ++lo;
    *tap = lo;
    int64_t start = seg[lo] + (int64_t)(chunk - cum[lo]) * L;
    int64_t left = seg[lo + 1] - start;
    *t0 = start;
    *rows = (int)(left < L ? left : L);
    return true;
}

constexpr int GL = 32;   // triplets per chunk
constexpr int GN = 64;   // output channels per block
constexpr int GK = 32;   // input channels per step

template <typename T, bool TRANSPOSE>
__global__ void __launch_bounds__(128) mvmr_sorted_kernel(
    const T *__restrict__ W, const T *__restrict__ feat, const int32_t *__restrict__ gather,
    const int32_t *__restrict__ scatter, const int64_t *__restrict__ seg, const int32_t *__restrict__ cum,
    float *__restrict__ acc, int K, int G, int C, int M) {
    __shared__ float xs[GL][GK + 1];
    __shared__ float ws[GK][GN + 1];
    __shared__ int32_t s_gather[GL], s_scatter[GL];
    int tap, rows;
    int64_t t0;
    if (!locate_chunk(cum, seg, K, GL, blockIdx.x, &tap, &t0, &rows)) return;
    const int g = blockIdx.z;
    const int inw = TRANSPOSE ? M : C, outw = TRANSPOSE ? C : M;
    const int n0 = blockIdx.y * GN;
    const int tid = threadIdx.x;
    if (tid < GL) {
        s_gather[tid] = tid < rows ? gather[t0 + tid] : 0;
        s_scatter[tid] = tid < rows ? scatter[t0 + tid] : 0;
    }
    __syncthreads();
    const T *Wk = W + ((int64_t)tap * G + g) * C * M;
    const int ty = tid >> 4, tx = tid & 15;
    float a[4][4] = {};
    for (int k0 = 0; k0 < inw; k0 += GK) {
        for (int idx = tid; idx < GL * GK; idx += 128) {
            int r = idx / GK, kk = idx % GK;
            float v = 0.f;
            if (r < rows && k0 + kk < inw)
                v = to_f32(feat[((int64_t)s_gather[r] * G + g) * inw + k0 + kk]);
            xs[r][kk] = v;
        }
        for (int idx = tid; idx < GK * GN; idx += 128) {
            int kk, n;
            if (TRANSPOSE) { n = idx / GK; kk = idx % GK; } else { kk = idx / GN; n = idx % GN; }
            float v = 0.f;
            if (k0 + kk < inw && n0 + n < outw) {
                int64_t off = TRANSPOSE ? (int64_t)(n0 + n) * M + (k0 + kk) : (int64_t)(k0 + kk) * M + (n0 + n);
                v = to_f32(Wk[off]);
            }
            ws[kk][n] = v;
        }
        __syncthreads();
#pragma unroll 8
        for (int kk = 0; kk < GK; ++kk) {
            float xv[4], wv[4];
#pragma unroll
            for (int r = 0; r < 4; ++r) xv[r] = xs[ty * 4 + r][kk];
#pragma unroll
            for (int c = 0; c < 4; ++c) wv[c] = ws[kk][tx * 4 + c];
#pragma unroll
            for (int r = 0; r < 4; ++r)
#pragma unroll
                for (int c = 0; c < 4; ++c) a[r][c] = __fmaf_rn(xv[r], wv[c], a[r][c]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int r = 0; r < 4; ++r) {
        int row = ty * 4 + r;
        if (row >= rows) continue;
        float *dst = acc + ((int64_t)s_scatter[row] * G + g) * outw;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            int n = n0 + tx * 4 + c;
            if (n < outw) atomicAdd(dst + n, a[r][c]);
        }
    }
}

// one warp per triplet, taps in any order
template <typename T, bool TRANSPOSE>
__global__ void mvmr_unsorted_kernel(const T *__restrict__ W, const T *__restrict__ feat,
                                     const int32_t *__restrict__ gather, const int32_t *__restrict__ scatter,
                                     const int32_t *__restrict__ tap_idx, float *__restrict__ acc,
                                     int64_t Tn, int G, int C, int M) {
    int64_t t = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (t >= Tn) return;
    const int lane = threadIdx.x & 31;
    const int inw = TRANSPOSE ? M : C, outw = TRANSPOSE ? C : M;
    const int64_t k = tap_idx[t], src = gather[t], dst = scatter[t];
    for (int g = 0; g < G; ++g) {
        const T *Wk = W + (k * G + g) * C * M;
        const T *x = feat + (src * G + g) * inw;
        float *o = acc + (dst * G + g) * outw;
        for (int n = lane; n < outw; n += 32) {
            float s = 0.f;
            for (int c = 0; c < inw; ++c) {
                int64_t off = TRANSPOSE ? (int64_t)n * M + c : (int64_t)c * M + n;
                s = __fmaf_rn(to_f32(x[c]), to_f32(Wk[off]), s);
            }
            atomicAdd(o + n, s);
        }
    }
}

constexpr int VL = 128;  // triplets per chunk
constexpr int VT = 64;   // tile edge
constexpr int VS = 8;    // triplets per step

template <typename T>
__global__ void __launch_bounds__(256) vvor_sorted_kernel(
    const T *__restrict__ A, const int32_t *__restrict__ a_idx, const T *__restrict__ B,
    const int32_t *__restrict__ b_idx, const int64_t *__restrict__ seg, const int32_t *__restrict__ cum,
    float *__restrict__ acc, int n_o, int G, int Ma, int Cb) {
    __shared__ float as[VS][VT], bs[VS][VT];
    __shared__ int32_t s_a[VL], s_b[VL];
    int o, rows;
    int64_t t0;
    if (!locate_chunk(cum, seg, n_o, VL, blockIdx.x, &o, &t0, &rows)) return;
    const int g = blockIdx.z;
    const int tiles_c = (Cb + VT - 1) / VT;
    const int m0 = (blockIdx.y / tiles_c) * VT, c0 = (blockIdx.y % tiles_c) * VT;
    const int tid = threadIdx.x;
    if (tid < VL) {
        s_a[tid] = tid < rows ? a_idx[t0 + tid] : 0;
        s_b[tid] = tid < rows ? b_idx[t0 + tid] : 0;
    }
    __syncthreads();
    const int ty = tid >> 4, tx = tid & 15;
    float r[4][4] = {};
    for (int s0 = 0; s0 < rows; s0 += VS) {
        for (int idx = tid; idx < VS * VT; idx += 256) {
            int s = idx / VT, e = idx % VT;
            float va = 0.f, vb = 0.f;
            if (s0 + s < rows) {
                if (m0 + e < Ma) va = to_f32(A[((int64_t)s_a[s0 + s] * G + g) * Ma + m0 + e]);
                if (c0 + e < Cb) vb = to_f32(B[((int64_t)s_b[s0 + s] * G + g) * Cb + c0 + e]);
            }
            as[s][e] = va;
            bs[s][e] = vb;
        }
        __syncthreads();
#pragma unroll
        for (int s = 0; s < VS; ++s) {
            float av[4], bv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) av[i] = as[s][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) bv[j] = bs[s][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) r[i][j] = __fmaf_rn(av[i], bv[j], r[i][j]);
        }
        __syncthreads();
    }
    float *dst = acc + ((int64_t)o * G + g) * Ma * Cb;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        int m = m0 + ty * 4 + i;
        if (m >= Ma) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            int c = c0 + tx * 4 + j;
            if (c < Cb) atomicAdd(dst + (int64_t)m * Cb + c, r[i][j]);
        }
    }
}

template <typename T>
__global__ void vvor_unsorted_kernel(const T *__restrict__ A, const int32_t *__restrict__ a_idx,
                                     const T *__restrict__ B, const int32_t *__restrict__ b_idx,
                                     const int32_t *__restrict__ o_idx, float *__restrict__ acc,
                                     int64_t Tn, int G, int Ma, int Cb) {
    int64_t t = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (t >= Tn) return;
    const int lane = threadIdx.x & 31;
    const int64_t ia = a_idx[t], ib = b_idx[t], io = o_idx[t];
    for (int g = 0; g < G; ++g) {
        const T *a = A + (ia * G + g) * Ma;
        const T *b = B + (ib * G + g) * Cb;
        float *o = acc + (io * G + g) * Ma * Cb;
        for (int m = 0; m < Ma; ++m) {
            float am = to_f32(a[m]);
            for (int c = lane; c < Cb; c += 32) atomicAdd(o + (int64_t)m * Cb + c, am * to_f32(b[c]));
        }
    }
}

template <typename T>
__global__ void round_kernel(const float *__restrict__ acc, T *__restrict__ out, int64_t n) {
    int64_t i = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) * 4;
    if (i + 3 < n) {
        float4 v = *reinterpret_cast<const float4 *>(acc + i);
        out[i] = from_f32<T>(v.x);
        out[i + 1] = from_f32<T>(v.y);
        out[i + 2] = from_f32<T>(v.z);
        out[i + 3] = from_f32<T>(v.w);
    } else {
        for (; i < n; ++i) out[i] = from_f32<T>(acc[i]);
    }
}

template <typename T>
int mvmr_generic_t(const MvmrArgs &a, cudaStream_t stream) {
    const T *W = (const T *)a.weight, *feat = (const T *)a.feat;
    const int outw = a.transpose ? a.C : a.M;
    if (a.seg_offs) {
        chunk_table_kernel<<<1, 128, 0, stream>>>(a.seg_offs, a.K, GL, a.chunk_table);
        PCX_LAUNCH_CHECK();
        prof_begin(a.transpose ? "mvmr_sorted_kernel(dgrad)" : "mvmr_sorted_kernel(fwd)", stream);
        int64_t upper = (a.T + GL - 1) / GL + a.K;
        dim3 grid((unsigned)upper, (unsigned)((outw + GN - 1) / GN), (unsigned)a.G);
        if (a.transpose)
            mvmr_sorted_kernel<T, true><<<grid, 128, 0, stream>>>(W, feat, a.gather, a.scatter, a.seg_offs, a.chunk_table, a.acc, a.K, a.G, a.C, a.M);
        else
            mvmr_sorted_kernel<T, false><<<grid, 128, 0, stream>>>(W, feat, a.gather, a.scatter, a.seg_offs, a.chunk_table, a.acc, a.K, a.G, a.C, a.M);
    } else {
        unsigned blocks = (unsigned)((a.T + 7) / 8);
        if (a.transpose)
            mvmr_unsorted_kernel<T, true><<<blocks, 256, 0, stream>>>(W, feat, a.gather, a.scatter, a.tap_idx, a.acc, a.T, a.G, a.C, a.M);
        else
            mvmr_unsorted_kernel<T, false><<<blocks, 256, 0, stream>>>(W, feat, a.gather, a.scatter, a.tap_idx, a.acc, a.T, a.G, a.C, a.M);
    }
    if (a.seg_offs) prof_end(stream);
    PCX_LAUNCH_CHECK();
    return PCX_OK;
}

template <typename T>
int vvor_generic_t(const VvorArgs &a, cudaStream_t stream) {
    const T *A = (const T *)a.a, *B = (const T *)a.b;
    if (a.seg_offs) {
        chunk_table_kernel<<<1, 128, 0, stream>>>(a.seg_offs, (int)a.n_o, VL, a.chunk_table);
        PCX_LAUNCH_CHECK();
        int64_t upper = (a.T + VL - 1) / VL + a.n_o;
        int tiles = ((a.Ma + VT - 1) / VT) * ((a.Cb + VT - 1) / VT);
        dim3 grid((unsigned)upper, (unsigned)tiles, (unsigned)a.G);
        prof_begin("vvor_sorted_kernel", stream);
        vvor_sorted_kernel<T><<<grid, 256, 0, stream>>>(A, a.a_idx, B, a.b_idx, a.seg_offs, a.chunk_table, a.acc, (int)a.n_o, a.G, a.Ma, a.Cb);
    } else {
        unsigned blocks = (unsigned)((a.T + 7) / 8);
        vvor_unsorted_kernel<T><<<blocks, 256, 0, stream>>>(A, a.a_idx, B, a.b_idx, a.o_idx, a.acc, a.T, a.G, a.Ma, a.Cb);
    }
    if (a.seg_offs) prof_end(stream);
    PCX_LAUNCH_CHECK();
    return PCX_OK;
}

}  // namespace

int mvmr_generic(const MvmrArgs &a, cudaStream_t stream) {
    switch (a.dtype) {
        case PCX_F32: return mvmr_generic_t<float>(a, stream);
        case PCX_F16: return mvmr_generic_t<__half>(a, stream);
        case PCX_BF16: return mvmr_generic_t<__nv_bfloat16>(a, stream);
    }
    PCX_FAIL(PCX_E_DTYPE, "unsupported dtype %d", a.dtype);
}

int vvor_generic(const VvorArgs &a, cudaStream_t stream) {
    switch (a.dtype) {
        case PCX_F32: return vvor_generic_t<float>(a, stream);
        case PCX_F16: return vvor_generic_t<__half>(a, stream);
        case PCX_BF16: return vvor_generic_t<__nv_bfloat16>(a, stream);
    }
    PCX_FAIL(PCX_E_DTYPE, "unsupported dtype %d", a.dtype);
}

int round_accumulator(const float *acc, void *out, int64_t n, int dtype, cudaStream_t stream) {
    if (n == 0) return PCX_OK;
    unsigned blocks = (unsigned)((n / 4 + 255) / 256 + 1);
    if (dtype == PCX_F16) round_kernel<__half><<<blocks, 256, 0, stream>>>(acc, (__half *)out, n);
    else if (dtype == PCX_BF16) round_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(acc, (__nv_bfloat16 *)out, n);
    else PCX_FAIL(PCX_E_DTYPE, "round_accumulator: dtype %d", dtype);
    PCX_LAUNCH_CHECK();
    return PCX_OK;
}

}  // namespace pcx
