// Thread-local error message, version, launch counter and the optional
// per-kernel event timer of the C-ABI library.
#include <stdarg.h>

#include <atomic>
#include <vector>

#include "common.cuh"

namespace pcx {
static thread_local char g_error[512] = "";

void set_error(const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
}

std::atomic<long long> g_launches{0};

struct ProfRecord {
    const char *name;
    cudaEvent_t start, stop;
};
static bool g_prof_on = false;
static std::vector<ProfRecord> g_prof;
static size_t g_prof_used = 0;
static constexpr size_t kProfCapacity = 1 << 14;

// Brackets the dominant kernel of an entry point with CUDA events recorded on
// the launch stream.  No effect unless pcx_profile_enable(1) was called.
void prof_begin(const char *name, cudaStream_t stream) {
    if (!g_prof_on || g_prof_used >= kProfCapacity) return;
    if (g_prof_used == g_prof.size()) {
        ProfRecord r{name, nullptr, nullptr};
        if (cudaEventCreate(&r.start) != cudaSuccess || cudaEventCreate(&r.stop) != cudaSuccess) return;
        g_prof.push_back(r);
    }
    g_prof[g_prof_used].name = name;
    cudaEventRecord(g_prof[g_prof_used].start, stream);
}

void prof_end(cudaStream_t stream) {
    if (!g_prof_on || g_prof_used >= g_prof.size()) return;
    cudaEventRecord(g_prof[g_prof_used].stop, stream);
    ++g_prof_used;
}
}  // namespace pcx

extern "C" {
int pcx_version(void) { return 10100; }
const char *pcx_last_error_string(void) { return pcx::g_error; }

long long pcx_launch_count(int reset) {
    long long v = pcx::g_launches.load();
    if (reset) pcx::g_launches.store(0);
    return v;
}

int pcx_profile_enable(int on) {
    pcx::g_prof_on = on != 0;
    pcx::g_prof_used = 0;
    return PCX_OK;
}

int pcx_profile_count(void) { return (int)pcx::g_prof_used; }

int pcx_profile_get(int index, const char **name, float *milliseconds) {
    if (index < 0 || (size_t)index >= pcx::g_prof_used || !name || !milliseconds)
        PCX_FAIL(PCX_E_ARG, "pcx_profile_get: bad index %d", index);
    auto &r = pcx::g_prof[index];
    PCX_CUDA(cudaEventSynchronize(r.stop));
    PCX_CUDA(cudaEventElapsedTime(milliseconds, r.start, r.stop));
    *name = r.name;
    return PCX_OK;
}
}
