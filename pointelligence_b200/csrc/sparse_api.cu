// extern "C" entry points of the sparse engines: argument checks, workspace
// carving, engine selection (tcgen05 tensor path vs CUDA-core path) and the
// single rounding of the fp32 accumulator into the output element type.
#include <algorithm>

#include "sparse_kernels.cuh"

namespace pcx {
int read_device_status(unsigned int *h_status, bool clear, cudaStream_t stream);

namespace {

struct MvmrWs {
    float *acc;
    int32_t *chunk_table;
};

size_t carve_mvmr(void *ws, int64_t n_out, int K, int G, int C, int M, int transpose, int dtype, MvmrWs *out) {
    Carver c(ws);
    MvmrWs w;
    const int outw = transpose ? C : M;
    w.acc = c.take<float>(dtype == PCX_F32 ? 1 : (size_t)n_out * G * outw);
    w.chunk_table = c.take<int32_t>((size_t)K + 1);
    if (out) *out = w;
    return c.off;
}

struct VvorWs {
    float *acc;
    int32_t *chunk_table;
};

size_t carve_vvor(void *ws, int64_t n_o, int G, int Ma, int Cb, int dtype, VvorWs *out) {
    Carver c(ws);
    VvorWs w;
    w.acc = c.take<float>(dtype == PCX_F32 ? 1 : (size_t)n_o * G * Ma * Cb);
    w.chunk_table = c.take<int32_t>((size_t)n_o + 1);
    if (out) *out = w;
    return c.off;
}

int force_engine() {
    static int v = -1;
    if (v < 0) {
        const char *e = getenv("PCX_ENGINE");
        v = e ? atoi(e) : 0;
        if (v < 0 || v > 2) v = 0;
    }
    return v;
}

}  // namespace
}  // namespace pcx

using namespace pcx;

extern "C" {

size_t pcx_mvmr_workspace_bytes(int64_t n_out, int K, int G, int C, int M, int transpose, int dtype) {
    if (n_out < 0 || K <= 0 || G <= 0 || C <= 0 || M <= 0) return 0;
    uint64_t checked = 0;
    if (!product_within((uint64_t)1 << 46, &checked, n_out, G, std::max(C, M))) return 0;
    return carve_mvmr(nullptr, n_out, K, G, C, M, transpose, dtype, nullptr);
}

int pcx_mvmr(const void *d_weight, const void *d_feat, const int32_t *d_gather, const int32_t *d_scatter,
             const int64_t *d_seg_offs, const int32_t *d_tap_idx, void *d_out, int64_t T, int64_t n_feat,
             int64_t n_out, int K, int G, int C, int M, int transpose, int dtype, int engine, void *d_ws,
             size_t ws_bytes, void *stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    if (T < 0 || n_feat < 0 || n_out < 0 || K <= 0 || G <= 0 || C <= 0 || M <= 0)
        PCX_FAIL(PCX_E_ARG, "pcx_mvmr: negative or zero size (T=%lld n_feat=%lld n_out=%lld K=%d G=%d C=%d M=%d)",
                 (long long)T, (long long)n_feat, (long long)n_out, K, G, C, M);
    if (dtype != PCX_F32 && dtype != PCX_F16 && dtype != PCX_BF16) PCX_FAIL(PCX_E_DTYPE, "pcx_mvmr: unsupported dtype %d", dtype);
    const bool fan_in_one = (engine & PCX_ENGINE_FLAG_FAN_IN_ONE) != 0;
    engine &= ~PCX_ENGINE_FLAG_FAN_IN_ONE;
    if (engine < 0 || engine > 2) PCX_FAIL(PCX_E_ARG, "pcx_mvmr: unknown engine %d", engine);
    if (fan_in_one && T != n_out) PCX_FAIL(PCX_E_ARG, "pcx_mvmr: fan-in 1 means one triplet per output row (T=%lld, n_out=%lld)", (long long)T, (long long)n_out);
    if (!d_weight || (n_out > 0 && !d_out) || !d_ws) PCX_FAIL(PCX_E_ARG, "pcx_mvmr: null pointer");
    if (T > 0 && (!d_feat || !d_gather || !d_scatter)) PCX_FAIL(PCX_E_ARG, "pcx_mvmr: null pointer");
    if (T > 0 && !d_seg_offs && !d_tap_idx) PCX_FAIL(PCX_E_ARG, "pcx_mvmr: either d_seg_offs or d_tap_idx is required");
    if ((uintptr_t)d_ws % 256) PCX_FAIL(PCX_E_ALIGN, "pcx_mvmr: workspace must be 256-byte aligned");
    if (n_feat > INT32_MAX || n_out > INT32_MAX) PCX_FAIL(PCX_E_UNSUPPORTED, "pcx_mvmr: more than 2^31-1 rows");
    uint64_t checked = 0;
    if (!product_within((uint64_t)1 << 46, &checked, n_out, G, std::max(C, M)) ||
        !product_within((uint64_t)1 << 46, &checked, K, G, C, M))
        PCX_FAIL(PCX_E_CAPACITY, "pcx_mvmr: n_out*G*width or K*G*C*M is beyond 2^46 elements");
    MvmrWs w;
    size_t need = carve_mvmr(d_ws, n_out, K, G, C, M, transpose, dtype, &w);
    if (ws_bytes < need) PCX_FAIL(PCX_E_CAPACITY, "pcx_mvmr: workspace %zu < %zu bytes", ws_bytes, need);
    const int outw = transpose ? C : M;
    const int64_t out_elems = n_out * G * outw;
    if (out_elems == 0) return PCX_OK;

    MvmrArgs a = {};
    a.weight = d_weight, a.feat = d_feat, a.gather = d_gather, a.scatter = d_scatter;
    a.seg_offs = d_seg_offs, a.tap_idx = d_tap_idx;
    a.acc = dtype == PCX_F32 ? (float *)d_out : w.acc;
    a.chunk_table = w.chunk_table;
    a.T = T, a.n_feat = n_feat, a.n_out = n_out;
    a.K = K, a.G = G, a.C = C, a.M = M, a.transpose = transpose ? 1 : 0, a.dtype = dtype;
    if (force_engine()) engine = force_engine();
    if (fan_in_one && T > 0 && engine != PCX_ENGINE_CUDA_CORE && mvmr_tensor_supported(a) && ((uintptr_t)d_out & 15) == 0) {
        // every output row has exactly one triplet: the tensor kernel stores the rounded rows
        // itself -- no accumulator to clear, no reductions, no rounding pass
        a.out_rows = d_out;
        return mvmr_tensor(a, stream);
    }
    PCX_CUDA(cudaMemsetAsync(a.acc, 0, (size_t)out_elems * sizeof(float), stream));
    if (T > 0) {
        bool tensor_ok = mvmr_tensor_supported(a);
        if (engine == PCX_ENGINE_TENSOR && !tensor_ok)
            PCX_FAIL(PCX_E_UNSUPPORTED, "pcx_mvmr: tensor engine needs fp16/bf16, G=1, tap-sorted triplets and channel counts that are multiples of 16 in [16,256]");
        int rc = (engine != PCX_ENGINE_CUDA_CORE && tensor_ok) ? mvmr_tensor(a, stream) : mvmr_generic(a, stream);
        if (rc != PCX_OK) return rc;
    }
    if (dtype != PCX_F32) return round_accumulator(a.acc, d_out, out_elems, dtype, stream);
    return PCX_OK;
}

size_t pcx_vvor_workspace_bytes(int64_t n_o, int G, int Ma, int Cb, int dtype) {
    if (n_o < 0 || G <= 0 || Ma <= 0 || Cb <= 0) return 0;
    uint64_t checked = 0;
    if (!product_within((uint64_t)1 << 46, &checked, n_o, G, Ma, Cb)) return 0;
    return carve_vvor(nullptr, n_o, G, Ma, Cb, dtype, nullptr);
}

int pcx_vvor(const void *d_a, const int32_t *d_a_idx, const void *d_b, const int32_t *d_b_idx,
             const int64_t *d_seg_offs, const int32_t *d_o_idx, void *d_out, int64_t T, int64_t n_a,
             int64_t n_b, int64_t n_o, int G, int Ma, int Cb, int dtype, int engine, void *d_ws,
             size_t ws_bytes, void *stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    if (T < 0 || n_a < 0 || n_b < 0 || n_o < 0 || G <= 0 || Ma <= 0 || Cb <= 0)
        PCX_FAIL(PCX_E_ARG, "pcx_vvor: negative or zero size");
    if (dtype != PCX_F32 && dtype != PCX_F16 && dtype != PCX_BF16) PCX_FAIL(PCX_E_DTYPE, "pcx_vvor: unsupported dtype %d", dtype);
    if (engine < 0 || engine > 2) PCX_FAIL(PCX_E_ARG, "pcx_vvor: unknown engine %d", engine);
    if ((n_o > 0 && !d_out) || !d_ws) PCX_FAIL(PCX_E_ARG, "pcx_vvor: null pointer");
    if (T > 0 && (!d_a || !d_b || !d_a_idx || !d_b_idx)) PCX_FAIL(PCX_E_ARG, "pcx_vvor: null pointer");
    if (T > 0 && !d_seg_offs && !d_o_idx) PCX_FAIL(PCX_E_ARG, "pcx_vvor: either d_seg_offs or d_o_idx is required");
    if ((uintptr_t)d_ws % 256) PCX_FAIL(PCX_E_ALIGN, "pcx_vvor: workspace must be 256-byte aligned");
    if (n_a > INT32_MAX || n_b > INT32_MAX || n_o > INT32_MAX) PCX_FAIL(PCX_E_UNSUPPORTED, "pcx_vvor: more than 2^31-1 rows");
    uint64_t checked = 0;
    if (!product_within((uint64_t)1 << 46, &checked, n_o, G, Ma, Cb))
        PCX_FAIL(PCX_E_CAPACITY, "pcx_vvor: n_o*G*Ma*Cb is beyond 2^46 elements");
    VvorWs w;
    size_t need = carve_vvor(d_ws, n_o, G, Ma, Cb, dtype, &w);
    if (ws_bytes < need) PCX_FAIL(PCX_E_CAPACITY, "pcx_vvor: workspace %zu < %zu bytes", ws_bytes, need);
    const int64_t out_elems = n_o * G * Ma * Cb;
    if (out_elems == 0) return PCX_OK;

    VvorArgs a = {};
    a.a = d_a, a.a_idx = d_a_idx, a.b = d_b, a.b_idx = d_b_idx, a.seg_offs = d_seg_offs, a.o_idx = d_o_idx;
    a.acc = dtype == PCX_F32 ? (float *)d_out : w.acc;
    a.chunk_table = w.chunk_table;
    a.T = T, a.n_a = n_a, a.n_b = n_b, a.n_o = n_o, a.G = G, a.Ma = Ma, a.Cb = Cb, a.dtype = dtype;
    PCX_CUDA(cudaMemsetAsync(a.acc, 0, (size_t)out_elems * sizeof(float), stream));
    if (T > 0) {
        if (force_engine()) engine = force_engine();
        bool tensor_ok = vvor_tensor_supported(a);
        if (engine == PCX_ENGINE_TENSOR && !tensor_ok)
            PCX_FAIL(PCX_E_UNSUPPORTED, "pcx_vvor: tensor engine needs fp16/bf16, G=1, sorted output index and channel counts that are multiples of 16 in [16,256]");
        int rc = (engine != PCX_ENGINE_CUDA_CORE && tensor_ok) ? vvor_tensor(a, stream) : vvor_generic(a, stream);
        if (rc != PCX_OK) return rc;
    }
    if (dtype != PCX_F32) return round_accumulator(a.acc, d_out, out_elems, dtype, stream);
    return PCX_OK;
}

int pcx_device_status(unsigned int *h_status, int clear, void *stream) {
    if (!h_status) PCX_FAIL(PCX_E_ARG, "pcx_device_status: null pointer");
    return read_device_status(h_status, clear != 0, (cudaStream_t)stream);
}

}  // extern "C"
