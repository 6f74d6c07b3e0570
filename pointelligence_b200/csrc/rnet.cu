// Residual R-net selector of the full-cover strided rulebook, on the device.
//
// Given the points no initial centre covers, with their neighbour lists within R (query-major,
// self included), centres are chosen in rounds: every still-active point has a priority
// (most active neighbours first, then farthest from its stride cell's initial centre, then lowest
// source index); a point whose priority is the best among its active neighbours becomes a centre and
// retires its whole neighbourhood.  The result is a maximal set of points pairwise farther apart
// than R that covers every input point -- the same set, point for point, as the reference's
// layers/triplets.py:156-232, which ranks all points with three stable sorts per round and takes a
// scatter-min over the edges; comparing the priority tuples directly gives the same winners
// without any sort.  One call runs a batch of rounds (three small kernels each) and hands the
// number of points still active after each of them back in one copy.
#include "common.cuh"

namespace pcx {
namespace {

// squared distance to the initial centre with one rounding per operation, in the order
// ((dx^2 + dy^2) + dz^2)
__global__ void rnet_far_kernel(const float *__restrict__ points, const float *__restrict__ centres,
                                const int64_t *__restrict__ centre_of, int64_t n, float *far) {
    const int64_t v = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (v >= n) return;
    const float *p = points + 3 * v, *c = centres + 3 * centre_of[v];
    const float dx = __fsub_rn(p[0], c[0]), dy = __fsub_rn(p[1], c[1]), dz = __fsub_rn(p[2], c[2]);
    far[v] = __fadd_rn(__fadd_rn(__fmul_rn(dx, dx), __fmul_rn(dy, dy)), __fmul_rn(dz, dz));
}

__global__ void rnet_gain_kernel(const int64_t *__restrict__ nb, const int64_t *__restrict__ offs,
                                 const uint8_t *__restrict__ active, int64_t n, int32_t *gain) {
    const int64_t v = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (v >= n) return;
    int32_t g = 0;
    if (active[v])
        for (int64_t e = offs[v]; e < offs[v + 1]; ++e) g += active[nb[e]];
    gain[v] = g;
}

// true when a comes before b: more active neighbours, then farther from its initial centre, then lower source index
__device__ __forceinline__ bool before(int32_t ga, float fa, int64_t sa, int32_t gb, float fb, int64_t sb) {
    if (ga != gb) return ga > gb;
    if (fa != fb) return fa > fb;
    return sa < sb;
}

__global__ void rnet_pick_kernel(const int64_t *__restrict__ nb, const int64_t *__restrict__ offs,
                                 const uint8_t *__restrict__ active, const int32_t *__restrict__ gain,
                                 const float *__restrict__ far, const int64_t *__restrict__ source, int64_t n,
                                 uint8_t *pick, uint8_t *chosen) {
    const int64_t v = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (v >= n) return;
    bool best = active[v] != 0;
    if (best) {
        const int32_t g = gain[v];
        const float f = far[v];
        const int64_t s = source[v];
        for (int64_t e = offs[v]; e < offs[v + 1] && best; ++e) {
            const int64_t p = nb[e];
            if (p != v && active[p] && before(gain[p], far[p], source[p], g, f, s)) best = false;
        }
    }
    pick[v] = best;
    if (best) chosen[v] = 1;
}

__global__ void rnet_retire_kernel(const int64_t *__restrict__ nb, const int64_t *__restrict__ offs,
                                   const uint8_t *__restrict__ pick, int64_t n, uint8_t *active) {
    const int64_t v = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (v >= n || !pick[v]) return;
    for (int64_t e = offs[v]; e < offs[v + 1]; ++e) active[nb[e]] = 0;
}

__global__ void rnet_count_kernel(const uint8_t *__restrict__ active, int64_t n, int32_t *remaining) {
    const int64_t v = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const unsigned m = __ballot_sync(0xffffffffu, v < n && active[v]);
    if ((threadIdx.x & 31) == 0 && m) atomicAdd(remaining, __popc(m));
}

}  // namespace
}  // namespace pcx

using namespace pcx;

extern "C" {

size_t pcx_rnet_workspace_bytes(int64_t n, int rounds) {
    if (n < 0 || rounds <= 0) return 0;
    Carver c(nullptr);
    c.take<int32_t>((size_t)n);       // gain
    c.take<uint8_t>((size_t)n);       // pick
    c.take<int32_t>((size_t)rounds);  // remaining per round
    return c.off;
}

int pcx_rnet_far(const float *d_points, const float *d_centres, const int64_t *d_centre_of, int64_t n, float *d_far,
                 void *stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    if (n < 0 || (n > 0 && (!d_points || !d_centres || !d_centre_of || !d_far)))
        PCX_FAIL(PCX_E_ARG, "pcx_rnet_far: null pointer or negative size");
    if (n == 0) return PCX_OK;
    rnet_far_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(d_points, d_centres, d_centre_of, n, d_far);
    PCX_LAUNCH_CHECK();
    return PCX_OK;
}

int pcx_rnet_rounds(const int64_t *d_neighbors, const int64_t *d_offsets, const float *d_far, const int64_t *d_source,
                    int64_t n, int rounds, uint8_t *d_active, uint8_t *d_chosen, int32_t *h_remaining, void *d_ws,
                    size_t ws_bytes, void *stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    if (n <= 0 || rounds <= 0 || rounds > 64) PCX_FAIL(PCX_E_ARG, "pcx_rnet_rounds: n must be positive, rounds within 1..64");
    if (!d_neighbors || !d_offsets || !d_far || !d_source || !d_active || !d_chosen || !h_remaining || !d_ws)
        PCX_FAIL(PCX_E_ARG, "pcx_rnet_rounds: null pointer");
    if ((uintptr_t)d_ws % 256) PCX_FAIL(PCX_E_ALIGN, "pcx_rnet_rounds: workspace must be 256-byte aligned");
    if (ws_bytes < pcx_rnet_workspace_bytes(n, rounds))
        PCX_FAIL(PCX_E_CAPACITY, "pcx_rnet_rounds: workspace %zu < %zu bytes", ws_bytes, pcx_rnet_workspace_bytes(n, rounds));
    Carver c(d_ws);
    int32_t *gain = c.take<int32_t>((size_t)n);
    uint8_t *pick = c.take<uint8_t>((size_t)n);
    int32_t *remaining = c.take<int32_t>((size_t)rounds);
    const unsigned blocks = (unsigned)((n + 255) / 256);
    PCX_CUDA(cudaMemsetAsync(remaining, 0, (size_t)rounds * sizeof(int32_t), stream));
    for (int r = 0; r < rounds; ++r) {
        rnet_gain_kernel<<<blocks, 256, 0, stream>>>(d_neighbors, d_offsets, d_active, n, gain);
        PCX_LAUNCH_CHECK();
        rnet_pick_kernel<<<blocks, 256, 0, stream>>>(d_neighbors, d_offsets, d_active, gain, d_far, d_source, n, pick, d_chosen);
        PCX_LAUNCH_CHECK();
        rnet_retire_kernel<<<blocks, 256, 0, stream>>>(d_neighbors, d_offsets, pick, n, d_active);
        PCX_LAUNCH_CHECK();
        rnet_count_kernel<<<blocks, 256, 0, stream>>>(d_active, n, remaining + r);
        PCX_LAUNCH_CHECK();
    }
    PCX_CUDA(cudaMemcpyAsync(h_remaining, remaining, (size_t)rounds * sizeof(int32_t), cudaMemcpyDeviceToHost, stream));
    PCX_CUDA(cudaStreamSynchronize(stream));
    return PCX_OK;
}

}  // extern "C"
