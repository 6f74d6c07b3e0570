// Per-output lists of a tap-sorted rulebook, for the dense-tap schedule: the
// triplets regrouped by scatter row (stable), each as the row `gather * K + tap`
// of the all-taps product it names, plus the list length of every output row.
// The reference has no counterpart (it never leaves the scatter schedule,
// sparse_engines/tig.py:1090-1206); max_pool3d's (j, num_neighbors) pair
// (layers/pooling.py:35-46) has the same shape.
#include <cub/cub.cuh>

#include "sparse_kernels.cuh"

namespace pcx {
namespace {

__global__ void ol_keys_kernel(const int32_t *__restrict__ scatter, const int32_t *__restrict__ gather,
                               const int64_t *__restrict__ seg, int64_t T, int K, uint32_t *keys, uint32_t *vals) {
    int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= T) return;
    int lo = 0, hi = K;   // tap = last k with seg[k] <= t
    while (hi - lo > 1) {
        int mid = (lo + hi) >> 1;
        if (seg[mid] <= t) lo = mid; else hi = mid;
    }
    keys[t] = (uint32_t)scatter[t];
    vals[t] = (uint32_t)gather[t] * (uint32_t)K + (uint32_t)lo;
}

// lengths[r] = number of sorted keys equal to r
__global__ void ol_lengths_kernel(const uint32_t *__restrict__ keys, int64_t T, int64_t n_out, int64_t *lengths) {
    int64_t r = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= n_out) return;
    int64_t lo = 0, hi = T;
    while (lo < hi) {
        int64_t mid = (lo + hi) >> 1;
        if (keys[mid] < (uint32_t)r) lo = mid + 1; else hi = mid;
    }
    int64_t first = lo;
    hi = T;
    while (lo < hi) {
        int64_t mid = (lo + hi) >> 1;
        if (keys[mid] <= (uint32_t)r) lo = mid + 1; else hi = mid;
    }
    lengths[r] = lo - first;
}

struct OlWs {
    uint32_t *keys_a, *keys_b, *vals_a;
    void *cub_tmp;
    size_t cub_bytes;
};

int bits_of(int64_t n) {
    int bits = 1;
    while (((int64_t)1 << bits) < n) ++bits;
    return bits;
}

size_t carve_ol(void *ws, int64_t T, int64_t n_out, OlWs *out) {
    Carver c(ws);
    OlWs w;
    w.keys_a = c.take<uint32_t>((size_t)T);
    w.keys_b = c.take<uint32_t>((size_t)T);
    w.vals_a = c.take<uint32_t>((size_t)T);
    size_t bytes = 0;
    cub::DeviceRadixSort::SortPairs(nullptr, bytes, (const uint32_t *)nullptr, (uint32_t *)nullptr,
                                    (const uint32_t *)nullptr, (uint32_t *)nullptr, (int)std::max<int64_t>(T, 1), 0,
                                    bits_of(n_out));
    w.cub_bytes = bytes;
    w.cub_tmp = c.take<char>(bytes);
    if (out) *out = w;
    return c.off;
}

bool sizes_ok(int64_t T, int64_t n_feat, int64_t n_out, int K) {
    return T > 0 && T <= INT32_MAX && n_out > 0 && n_out <= INT32_MAX && K > 0 && n_feat >= 0 &&
           n_feat * K <= INT32_MAX;
}

}  // namespace
}  // namespace pcx

using namespace pcx;

extern "C" {

size_t pcx_output_lists_workspace_bytes(int64_t T, int64_t n_out) {
    if (T <= 0 || n_out <= 0) return 0;
    return carve_ol(nullptr, T, n_out, nullptr);
}

int pcx_output_lists(const int32_t *d_scatter, const int32_t *d_gather, const int64_t *d_seg_offs, int64_t T, int K,
                     int64_t n_feat, int64_t n_out, int32_t *d_src, int64_t *d_lengths, void *d_ws, size_t ws_bytes,
                     void *stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    if (!sizes_ok(T, n_feat, n_out, K))
        PCX_FAIL(PCX_E_ARG, "pcx_output_lists: sizes out of range (T=%lld n_feat=%lld n_out=%lld K=%d; n_feat*K must fit int32)",
                 (long long)T, (long long)n_feat, (long long)n_out, K);
    if (!d_scatter || !d_gather || !d_seg_offs || !d_src || !d_lengths || !d_ws)
        PCX_FAIL(PCX_E_ARG, "pcx_output_lists: null pointer");
    if ((uintptr_t)d_ws % 256) PCX_FAIL(PCX_E_ALIGN, "pcx_output_lists: workspace must be 256-byte aligned");
    OlWs w;
    size_t need = carve_ol(d_ws, T, n_out, &w);
    if (ws_bytes < need) PCX_FAIL(PCX_E_CAPACITY, "pcx_output_lists: workspace %zu < %zu bytes", ws_bytes, need);
    const int TPB = 256;
    ol_keys_kernel<<<(unsigned)((T + TPB - 1) / TPB), TPB, 0, stream>>>(d_scatter, d_gather, d_seg_offs, T, K, w.keys_a,
                                                                       w.vals_a);
    PCX_LAUNCH_CHECK();
    size_t bytes = w.cub_bytes;
    PCX_CUDA(cub::DeviceRadixSort::SortPairs(w.cub_tmp, bytes, w.keys_a, w.keys_b, w.vals_a, (uint32_t *)d_src, (int)T, 0,
                                             bits_of(n_out), stream));
    ol_lengths_kernel<<<(unsigned)((n_out + TPB - 1) / TPB), TPB, 0, stream>>>(w.keys_b, T, n_out, d_lengths);
    PCX_LAUNCH_CHECK();
    return PCX_OK;
}

}  // extern "C"
