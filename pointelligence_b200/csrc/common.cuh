// Shared helpers of the C-ABI library: status reporting, launch checks,
// workspace carving, element-type conversion.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include <atomic>

#include "../../include/pointelligence_b200.h"

namespace pcx {

void set_error(const char *fmt, ...);
extern std::atomic<long long> g_launches;               // kernels launched by this library
void prof_begin(const char *name, cudaStream_t stream); // event timer around a dominant kernel
void prof_end(cudaStream_t stream);

#define PCX_FAIL(code, ...)            \
    do {                               \
        ::pcx::set_error(__VA_ARGS__); \
        return (code);                 \
    } while (0)

#define PCX_CUDA(expr)                                                          \
    do {                                                                        \
        cudaError_t _e = (expr);                                                \
        if (_e != cudaSuccess)                                                  \
            PCX_FAIL(PCX_E_LAUNCH, "%s failed: %s (%s:%d)", #expr,              \
                     cudaGetErrorString(_e), __FILE__, __LINE__);               \
    } while (0)

#define PCX_LAUNCH_CHECK()            \
    do {                              \
        ::pcx::g_launches.fetch_add(1); \
        PCX_CUDA(cudaGetLastError()); \
    } while (0)

static inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

// Bump allocator over a caller-owned workspace; every block 256-byte aligned.
struct Carver {
    char *base;
    size_t off;
    explicit Carver(void *p) : base(static_cast<char *>(p)), off(0) {}
    template <typename T>
    T *take(size_t count) {
        T *p = reinterpret_cast<T *>(base + off);
        off += align_up(count * sizeof(T), 256);
        return p;
    }
};

// Product of non-negative sizes; false when a factor is negative or the product exceeds `limit`
// (checked factor by factor, so it cannot wrap on the way).
static inline bool product_within(uint64_t limit, uint64_t *out, int64_t a, int64_t b = 1, int64_t c = 1, int64_t d = 1) {
    const int64_t f[4] = {a, b, c, d};
    uint64_t p = 1;
    for (int i = 0; i < 4; ++i) {
        if (f[i] < 0) return false;
        if (__builtin_mul_overflow(p, (uint64_t)f[i], &p) || p > limit) return false;
    }
    *out = p;
    return true;
}

static inline size_t elem_size(int dtype) { return dtype == PCX_F32 ? 4 : 2; }

template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T>
__device__ __forceinline__ T from_f32(float v);
template <>
__device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

static inline int num_sms() {
    static int cached = 0;
    if (!cached) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&cached, cudaDevAttrMultiProcessorCount, dev);
        if (cached <= 0) cached = 148;
    }
    return cached;
}

}  // namespace pcx
