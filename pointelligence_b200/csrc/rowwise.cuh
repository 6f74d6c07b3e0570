// Row-wise access helpers of the byte-bound kernels (norms, segment reductions):
// 16-byte vector loads / stores of VN consecutive channels converted to fp32, and
// the thread layout (vector column, row lane) they share.
#pragma once
#include "common.cuh"

namespace pcx {

template <typename T>
struct VecWidth { static constexpr int value = 16 / sizeof(T); };

// VN == 1: scalar access (any channel count, any alignment); VN == 16 / sizeof(T): one 16-byte access
template <typename T, int VN>
__device__ __forceinline__ void load_vec(const T *__restrict__ p, float *out) {
    if constexpr (VN == 1) {
        out[0] = to_f32<T>(p[0]);
    } else {
        const uint4 raw = *reinterpret_cast<const uint4 *>(p);
        const T *e = reinterpret_cast<const T *>(&raw);
#pragma unroll
        for (int i = 0; i < VN; ++i) out[i] = to_f32<T>(e[i]);
    }
}

template <typename T, int VN>
__device__ __forceinline__ void store_vec(T *__restrict__ p, const float *in) {
    if constexpr (VN == 1) {
        p[0] = from_f32<T>(in[0]);
    } else {
        uint4 raw;
        T *e = reinterpret_cast<T *>(&raw);
#pragma unroll
        for (int i = 0; i < VN; ++i) e[i] = from_f32<T>(in[i]);
        *reinterpret_cast<uint4 *>(p) = raw;
    }
}

// Thread layout over a block of rows: `vcb` vector columns side by side, blockDim / vcb
// row lanes; a thread keeps its vector column for the whole pass.
struct RowLayout {
    int vc_total;   // vector columns of a row (C / VN)
    int vcb;        // vector columns handled per pass (<= blockDim)
    int lanes;      // row lanes
    int vc, lane;   // this thread's column inside a pass and its row lane (lane >= lanes: idle)
    __device__ __forceinline__ RowLayout(int C, int VN) {
        vc_total = C / VN;
        vcb = vc_total < (int)blockDim.x ? vc_total : (int)blockDim.x;
        lanes = blockDim.x / vcb;
        vc = threadIdx.x % vcb;
        lane = threadIdx.x / vcb;
    }
};

// first segment s with offsets[s + 1] > row (offsets has S + 1 entries)
__device__ __forceinline__ int64_t segment_of_row(const int64_t *__restrict__ offsets, int64_t S, int64_t row) {
    int64_t lo = 0, hi = S;
    while (lo < hi) {
        int64_t mid = (lo + hi) >> 1;
        if (offsets[mid + 1] <= row) lo = mid + 1; else hi = mid;
    }
    return lo;
}

static inline bool vec_ok(int C, int dtype, std::initializer_list<const void *> ptrs) {
    const int vn = 16 / (int)elem_size(dtype);
    if (C % vn) return false;
    for (const void *p : ptrs)
        if (p && ((uintptr_t)p & 15)) return false;
    return true;
}

}  // namespace pcx
