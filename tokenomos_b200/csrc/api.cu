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

// ---- index checks of a debug build (checks.cuh) ------------------------------------------------
#ifdef TK_CHECKS
namespace {
constexpr int MAX_CHECKED_FILES = 32;
int (*g_check_set[MAX_CHECKED_FILES])(int, int);
int (*g_check_get[MAX_CHECKED_FILES])(int*);
int g_checked_files = 0;
}  // namespace

void tk_checks_register(int (*set)(int, int), int (*get)(int*)) {
    if (g_checked_files < MAX_CHECKED_FILES) {
        g_check_set[g_checked_files] = set;
        g_check_get[g_checked_files] = get;
        ++g_checked_files;
    }
}
#endif

// 1 if the library was built with index checks (-DTK_CHECKS), else 0.
TK_API int tk_checks_enabled() {
#ifdef TK_CHECKS
    return 1;
#else
    return 0;
#endif
}

// The sizes the checks compare against: pages of every paged pool, rows of every state tensor.
TK_API int tk_checks_set_bounds(int pages, int slots) {
#ifdef TK_CHECKS
    for (int i = 0; i < g_checked_files; ++i)
        if (g_check_set[i](pages, slots) != 0) {
            tk_set_error("checks_set_bounds: copying the bounds to the device failed");
            return -1;
        }
#endif
    (void)pages;
    (void)slots;
    return 0;
}

// out[0] = kernel * 8 + kind of index (TkCheckedKernel, TkCheckedIndex), out[1] = the index, of
// the first index a kernel found outside its pool since the last call; out[0] = 0 if none.
// Resets the words.
TK_API int tk_checks_status(int* out) {
    out[0] = out[1] = 0;
#ifdef TK_CHECKS
    for (int i = 0; i < g_checked_files; ++i) {
        int word[2] = {0, 0};
        if (g_check_get[i](word) != 0) {
            tk_set_error("checks_status: reading the word from the device failed");
            return -1;
        }
        if (word[0] != 0 && out[0] == 0) {
            out[0] = word[0];
            out[1] = word[1];
        }
    }
#endif
    return 0;
}
