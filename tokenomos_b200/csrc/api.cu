// Error channel and build identity of the kernel library.
#include <stdarg.h>
#include <stdio.h>

#include "common.cuh"

static thread_local char g_error[512] = "";

void tk_set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
}

// The message of the last failed call on this thread ("" if none).
TK_API const char* tk_last_error() { return g_error; }

// Compute capability the library was built for (sm_100a only).
TK_API int tk_built_for() { return 100; }

// 0 when the current device can run this library, else a negative code with a message.
TK_API int tk_check_device() {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) {
        tk_set_error("no CUDA device: %s", cudaGetErrorString(e));
        return -1;
    }
    cudaDeviceProp p;
    e = cudaGetDeviceProperties(&p, dev);
    if (e != cudaSuccess) {
        tk_set_error("cudaGetDeviceProperties: %s", cudaGetErrorString(e));
        return -1;
    }
    if (p.major != 10) {
        tk_set_error("device %s is sm_%d%d; this library holds sm_100a code only", p.name, p.major,
                     p.minor);
        return -1;
    }
    return 0;
}

static int g_pdl = 1;

bool tk_pdl_enabled() { return g_pdl != 0; }

// 1: kernels are launched with programmatic stream serialization (the default); 0: plain order.
TK_API int tk_set_pdl(int on) {
    g_pdl = on ? 1 : 0;
    return 0;
}
