// pcx_vvor_static_scratch: the weight-gradient reduction for callers that
// cannot hand the library a workspace.
//
// Some hosts of this library have no way to obtain device memory at the moment
// they need a weight gradient: code running inside another framework's
// allocator callback or inside a region where cudaMalloc is forbidden (it
// synchronises the device), plugins whose only device memory is the tensors
// they were given, or embedders that pre-plan every byte.  For them this entry
// point keeps the two scratch buffers VVOR needs -- the fp32 accumulator and
// the per-output chunk table -- in one file-scope __device__ array of fixed
// size.  Every GPU whose context loads the library carries that array
// (kStaticScratchBytes, about 8 MiB) until the process exits.
//
// The array's name in host code is only a host-side handle; the kernels get
// the device address that cudaGetSymbolAddress returns for the current device.
// That lookup happens on the first call made with a given device current, so
// make that first call outside any stream capture.
//
// All calls share the array: its previous contents are cleared as part of the
// call, and two calls that overlap on the GPU (different streams, or different
// host threads) race on it.  Serialise them.
#include <mutex>

#include "sparse_kernels.cuh"

namespace pcx {
namespace {

constexpr size_t kMaxAccumulatorFloats = size_t(1) << 21;   // 8 MiB of fp32 partial sums
constexpr size_t kMaxOutputs = 4095;                        // n_o; the chunk table holds n_o + 1 ints
constexpr size_t kTableBytes = (kMaxOutputs + 1) * sizeof(int32_t);
constexpr size_t kStaticScratchBytes = kMaxAccumulatorFloats * sizeof(float) + kTableBytes;

static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
std::mutex g_setup_mutex;
void *g_scratch_addr[kMaxDevices] = {};

// Device address of the array on the current device (looked up once per device).
int static_scratch_address(void **out) {
    int dev = 0;
    PCX_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) PCX_FAIL(PCX_E_UNSUPPORTED, "device ordinal %d is out of range", dev);
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (!g_scratch_addr[dev]) {
        void *ptr = nullptr;
        PCX_CUDA(cudaGetSymbolAddress(&ptr, g_static_scratch));
        if (!ptr) PCX_FAIL(PCX_E_LAUNCH, "cudaGetSymbolAddress returned a null address");
        g_scratch_addr[dev] = ptr;
    }
    *out = g_scratch_addr[dev];
    return PCX_OK;
}

}  // namespace
}  // namespace pcx

using namespace pcx;

extern "C" {

size_t pcx_vvor_static_scratch_max_elements(void) { return kMaxAccumulatorFloats; }

int pcx_vvor_static_scratch(const void *d_a, const int32_t *d_a_idx, const void *d_b, const int32_t *d_b_idx,
                            const int64_t *d_seg_offs, void *d_out, int64_t T, int64_t n_a, int64_t n_b,
                            int64_t n_o, int G, int Ma, int Cb, int dtype, void *stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    if (T < 0 || n_a < 0 || n_b < 0 || n_o <= 0 || G <= 0 || Ma <= 0 || Cb <= 0)
        PCX_FAIL(PCX_E_ARG, "pcx_vvor_static_scratch: negative or zero size");
    if (dtype != PCX_F32 && dtype != PCX_F16 && dtype != PCX_BF16)
        PCX_FAIL(PCX_E_DTYPE, "pcx_vvor_static_scratch: unsupported dtype %d", dtype);
    if (!d_out || !d_seg_offs) PCX_FAIL(PCX_E_ARG, "pcx_vvor_static_scratch: d_out and d_seg_offs are required");
    if (T > 0 && (!d_a || !d_b || !d_a_idx || !d_b_idx)) PCX_FAIL(PCX_E_ARG, "pcx_vvor_static_scratch: null pointer");
    if (n_a > INT32_MAX || n_b > INT32_MAX) PCX_FAIL(PCX_E_UNSUPPORTED, "pcx_vvor_static_scratch: more than 2^31-1 rows");
    uint64_t out_elems = 0;   // checked factor by factor: a product that wraps must not pass for a small one
    if ((size_t)n_o > kMaxOutputs || !product_within(kMaxAccumulatorFloats, &out_elems, n_o, G, Ma, Cb))
        PCX_FAIL(PCX_E_CAPACITY,
                 "pcx_vvor_static_scratch: output of %lld x %d x %d x %d elements exceeds the built-in scratch "
                 "(at most %zu elements and %zu rows); use pcx_vvor with a caller-owned workspace",
                 (long long)n_o, G, Ma, Cb, kMaxAccumulatorFloats, kMaxOutputs);
    void *scratch = nullptr;
    int rc = static_scratch_address(&scratch);
    if (rc != PCX_OK) return rc;

    VvorArgs a = {};
    a.a = d_a, a.a_idx = d_a_idx, a.b = d_b, a.b_idx = d_b_idx, a.seg_offs = d_seg_offs, a.o_idx = nullptr;
    a.acc = dtype == PCX_F32 ? (float *)d_out : (float *)scratch;
    a.chunk_table = (int32_t *)((unsigned char *)scratch + kMaxAccumulatorFloats * sizeof(float));
    a.T = T, a.n_a = n_a, a.n_b = n_b, a.n_o = n_o, a.G = G, a.Ma = Ma, a.Cb = Cb, a.dtype = dtype;
    // the accumulator still holds the previous call's sums
    PCX_CUDA(cudaMemsetAsync(a.acc, 0, out_elems * sizeof(float), stream));
    if (T > 0) {
        rc = vvor_tensor_supported(a) ? vvor_tensor(a, stream) : vvor_generic(a, stream);
        if (rc != PCX_OK) return rc;
    }
    if (dtype != PCX_F32) return round_accumulator(a.acc, d_out, (int64_t)out_elems, dtype, stream);
    return PCX_OK;
}

}  // extern "C"
