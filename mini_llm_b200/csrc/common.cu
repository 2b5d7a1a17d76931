// Error text of the last failed call, per host thread; library version.
#include "common.cuh"
#include <stdarg.h>

static thread_local char g_err[512] = "";

int mllm_fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

MLLM_EXPORT const char* mllm_last_error() { return g_err; }

MLLM_EXPORT int mllm_abi_version() { return 1; }

int g_mllm_pdl = 0;

// Programmatic dependent launch on (1) or off (0) for the kernels that support it.
MLLM_EXPORT int mllm_set_pdl(int on) {
    g_mllm_pdl = on ? 1 : 0;
    return 0;
}
