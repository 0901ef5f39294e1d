// Error reporting shared by all exported functions.
#include "common.cuh"

#include <stdarg.h>
#include <stdio.h>

static thread_local char g_last_error[512] = "";

void hymt2_set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
    va_end(ap);
}

int hymt2_check_launch(const char* what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        hymt2_set_error("%s: %s", what, cudaGetErrorString(e));
        return HYMT2_ERR_LAUNCH;
    }
    return HYMT2_OK;
}

HYMT2_API const char* hymt2_last_error() { return g_last_error; }

// Compiled for this architecture; the Python side checks it against the device.
HYMT2_API int hymt2_compiled_arch() { return 100; }

static int g_pdl_enabled = 1;
bool hymt2_pdl_enabled() { return g_pdl_enabled != 0; }

// Programmatic dependent launch of the decode kernels on (default) or off.
HYMT2_API void hymt2_set_pdl(int on) { g_pdl_enabled = on; }
