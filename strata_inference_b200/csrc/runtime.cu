// Error reporting shared by all exported launchers.
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>

#include "common.cuh"

static thread_local char g_error[512] = "";

void sib_set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
}

// After a launch: 0, or the CUDA error's code with its text recorded.
int sib_check_launch(const char* what) {
    cudaError_t e = cudaGetLastError();
    if (e == cudaSuccess) return 0;
    sib_set_error("%s: %s", what, cudaGetErrorString(e));
    return (int)e;
}

bool sib_chained_launches() {
    static int enabled = -1;
    if (enabled < 0) {
        const char* v = getenv("SIB_CHAINED_LAUNCH");
        enabled = (v && v[0] == '0') ? 0 : 1;
    }
    return enabled == 1;
}

SIB_EXPORT const char* sib_last_error() { return g_error; }

// The architecture this library was compiled for; the loader refuses any other.
SIB_EXPORT int sib_compiled_arch() {
#ifdef SIB_ARCH
    return SIB_ARCH;
#else
    return 0;
#endif
}
