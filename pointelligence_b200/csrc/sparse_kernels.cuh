// Argument blocks shared by the sparse-engine translation units.
#pragma once
#include "common.cuh"

namespace pcx {

struct MvmrArgs {
    const void *weight;      // (K,G,C,M)
    const void *feat;        // (n_feat, G*inw)
    const int32_t *gather;   // (T) rows of feat
    const int32_t *scatter;  // (T) rows of out
    const int64_t *seg_offs; // (K+1) or null
    const int32_t *tap_idx;  // (T) when seg_offs is null
    float *acc;              // (n_out, G*outw) fp32, zeroed by the caller
    void *out_rows;          // tensor engine, fan-in 1: the output itself, written row by row (acc unused)
    int32_t *chunk_table;    // (K+1) scratch of the CUDA-core engine
    int64_t T, n_feat, n_out;
    int K, G, C, M, transpose, dtype;
};

struct VvorArgs {
    const void *a;           // (n_a, G*Ma)
    const int32_t *a_idx;
    const void *b;           // (n_b, G*Cb)
    const int32_t *b_idx;
    const int64_t *seg_offs; // (n_o+1) or null
    const int32_t *o_idx;    // (T) when seg_offs is null
    float *acc;              // (n_o, G, Ma, Cb) fp32, zeroed by the caller
    int32_t *chunk_table;    // (n_o+1) scratch
    int64_t T, n_a, n_b, n_o;
    int G, Ma, Cb, dtype;
};

__global__ void chunk_table_kernel(const int64_t *__restrict__ seg, int K, int L, int32_t *cum);

int mvmr_generic(const MvmrArgs &a, cudaStream_t stream);
int vvor_generic(const VvorArgs &a, cudaStream_t stream);
int round_accumulator(const float *acc, void *out, int64_t n, int dtype, cudaStream_t stream);

bool mvmr_tensor_supported(const MvmrArgs &a);
bool vvor_tensor_supported(const VvorArgs &a);
int mvmr_tensor(const MvmrArgs &a, cudaStream_t stream);
int vvor_tensor(const VvorArgs &a, cudaStream_t stream);

}  // namespace pcx
