// Error reporting and library identification for the qmlb200 C ABI.
#include <stdarg.h>
#include <stdio.h>

#include "common.cuh"

namespace qmlb {

static thread_local char g_error[512] = "";

void set_error(const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
}

int check_launch(const char *what) {
    const cudaError_t e = cudaGetLastError();
    if (e == cudaSuccess) return QMLB_OK;
    set_error("%s: %s", what, cudaGetErrorString(e));
    return QMLB_ERR_CUDA;
}

}  // namespace qmlb

extern "C" const char *qmlb_last_error(void) { return qmlb::g_error; }

extern "C" int qmlb_version(void) { return 100; }
