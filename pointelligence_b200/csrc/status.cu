// Thread-local error message and version of the C-ABI library.
#include <stdarg.h>

#include "common.cuh"

namespace pcx {
static thread_local char g_error[512] = "";

void set_error(const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
}
}  // namespace pcx

extern "C" {
int pcx_version(void) { return 10000; }
const char *pcx_last_error_string(void) { return pcx::g_error; }
}
