// Device arithmetic shared by the geometry kernels.  Everything that decides membership is written
// with explicit round-to-nearest intrinsics (no FMA contraction unless the variant asks for it)
// because the results have to be bit-identical with the reference:
//   cell of a point       floor(p * inv)            internals/neighbors.py:613-619
//   predicate             sqrt((dx^2+dy^2)+dz^2)<=R sparse_engines/strided_grid_radius_triton_kernel.py:25-31,127
//   tap                   rint((p-q) / g), clamped  sparse_engines/strided_grid_radius_triton_kernel.py:71-92
#pragma once
#include "common.cuh"

namespace pcx {

int radius_variant();   // predicate arithmetic in use (see radius_accept); defined in geometry.cu

namespace geo {

__device__ __forceinline__ int cell_of(float v, float inv) { return (int)floorf(__fmul_rn(v, inv)); }
__device__ __forceinline__ int corner_of(float v, float r32, float inv) {
    return (int)floorf(__fmul_rn(__fsub_rn(v, r32), inv));
}


__device__ __forceinline__ uint64_t mix64(uint64_t x) {
    x ^= x >> 33;
    x *= 0xff51afd7ed558ccdULL;
    x ^= x >> 33;
    x *= 0xc4ceb9fe1a85ec53ULL;
    x ^= x >> 33;
    return x;
}

// Radius predicate  sqrt(dx*dx + dy*dy + dz*dz) <= R  in fp32.
//   variant 0  the expression as written: one rounding per operation (what the
//              reference computes under Triton's CPU interpreter and in numpy)
//   variant 1  the sum of squares contracted into fma(dz,dz, fma(dx,dx, dy*dy)),
//              which is what Triton compiles the expression to on a B200: on
//              1,048,576 pairs placed within 3 ulp of R the accepted sets were
//              identical, while variant 0 changed the neighbour count of 214 of the 4096 queries
//   variant 2  variant 1 with the approximate square root (same sets as 1 in
//              that measurement)
// Pairs farther than an ulp or two from R are classified identically by all.
__device__ __forceinline__ bool radius_accept(float qx, float qy, float qz, float4 p, float r32,
                                              int distance_type, int variant, float *dist_out) {
    float dx = __fsub_rn(qx, p.x), dy = __fsub_rn(qy, p.y), dz = __fsub_rn(qz, p.z);
    float d;
    if (distance_type == 0) {
        float s;
        if (variant == 0) {
            s = __fadd_rn(__fadd_rn(__fmul_rn(dx, dx), __fmul_rn(dy, dy)), __fmul_rn(dz, dz));
            d = __fsqrt_rn(s);
        } else {
            s = __fmaf_rn(dz, dz, __fmaf_rn(dx, dx, __fmul_rn(dy, dy)));
            if (variant == 1) d = __fsqrt_rn(s);
            else asm("sqrt.approx.ftz.f32 %0, %1;" : "=f"(d) : "f"(s));
        }
    } else {
        d = fmaxf(fmaxf(fabsf(dx), fabsf(dy)), fabsf(dz));
    }
    *dist_out = d;
    return d <= r32;
}

__device__ __forceinline__ int tap_of(float qx, float qy, float qz, float4 p, float g32, int K) {
    int half = K >> 1;
    int dx = __float2int_rn(__fdiv_rn(__fsub_rn(p.x, qx), g32));
    int dy = __float2int_rn(__fdiv_rn(__fsub_rn(p.y, qy), g32));
    int dz = __float2int_rn(__fdiv_rn(__fsub_rn(p.z, qz), g32));
    int kx = min(max(dx + half, 0), K - 1), ky = min(max(dy + half, 0), K - 1),
        kz = min(max(dz + half, 0), K - 1);
    return (kx * K + ky) * K + kz;
}

// The same tap without the three IEEE divisions where that is safe: rint(d / g) equals rint(d * (1 / g))
// unless the quotient lies within a few ulp of a half-integer, because the product differs from the
// correctly rounded quotient by at most about two ulp.  A component whose product is farther than
// 0.49 from its nearest integer (or large) is decided by the exact division, as in tap_of.
__device__ __forceinline__ int tap_axis_fast(float d, float g32, float inv_g) {
    const float t = __fmul_rn(d, inv_g);
    const float r = rintf(t);
    if (fabsf(t - r) > 0.49f || fabsf(t) > 4096.f) return __float2int_rn(__fdiv_rn(d, g32));
    return (int)r;
}
__device__ __forceinline__ int tap_of_fast(float qx, float qy, float qz, float4 p, float g32, float inv_g, int K) {
    const int half = K >> 1;
    const int dx = tap_axis_fast(__fsub_rn(p.x, qx), g32, inv_g), dy = tap_axis_fast(__fsub_rn(p.y, qy), g32, inv_g),
              dz = tap_axis_fast(__fsub_rn(p.z, qz), g32, inv_g);
    const int kx = min(max(dx + half, 0), K - 1), ky = min(max(dy + half, 0), K - 1), kz = min(max(dz + half, 0), K - 1);
    return (kx * K + ky) * K + kz;
}

}  // namespace geo
}  // namespace pcx
