// Index checks for a debug build (-DTK_CHECKS): every kernel that follows an index the host
// gave it into a pool (a page number from a block table, a state row, a row of a table) first
// compares it with the pool's size. An index outside is recorded, once, as (kernel, kind of
// index, value) in a word the host reads (tk_checks_status), and the kernel carries on with the
// null page or the null row instead of touching the address: nothing traps, the context stays
// usable, and the engine turns the word into an exception where it reads the other kernels'
// error words. This stands in for a memory checker where none can be run. The bounds are those
// of the pools the step function was built on (tk_checks_set_bounds); a plain build compiles
// the macros away.
//
// Without relocatable device code every source file has device variables of its own, so each
// keeps its copy of the bounds and of the word, and registers a setter and a getter with the
// library (api.cu), which fans a call out to all of them.
#pragma once

#include <cuda_runtime.h>

enum TkCheckedKernel : int {
    TK_K_GATHER = 1, TK_K_QK_ROPE = 2, TK_K_ATTN_GENERIC = 3, TK_K_ATTN_TILES = 4, TK_K_CONV = 5,
    TK_K_SKINNY_CONV = 6,
};
enum TkCheckedIndex : int { TK_CHK_PAGE = 1, TK_CHK_SLOT = 2, TK_CHK_ROW = 3 };

#ifdef TK_CHECKS

struct TkBounds {
    int pages, slots;
};
static __device__ TkBounds tk_bounds_d = {0x7fffffff, 0x7fffffff};
static __device__ int tk_check_word_d[2] = {0, 0};

// whether 0 <= v < bound; if not, the first such finding of this source file is recorded
__device__ __forceinline__ bool tk_check(int kernel, int what, long long v, long long bound) {
    if (v >= 0 && v < bound) return true;
    if (atomicCAS(&tk_check_word_d[0], 0, kernel * 8 + what) == 0) tk_check_word_d[1] = (int)v;
    return false;
}

#define TK_PAGE(kernel, page) (tk_check((kernel), TK_CHK_PAGE, (page), tk_bounds_d.pages) ? (page) : 0)
#define TK_SLOT(kernel, slot) (tk_check((kernel), TK_CHK_SLOT, (slot), tk_bounds_d.slots) ? (slot) : 0)
#define TK_ROW(kernel, row, bound) (tk_check((kernel), TK_CHK_ROW, (row), (bound)) ? (row) : 0)

void tk_checks_register(int (*set)(int, int), int (*get)(int*));

static int tk_checks_set_here(int pages, int slots) {
    const TkBounds b{pages, slots};
    return cudaMemcpyToSymbol(tk_bounds_d, &b, sizeof(b)) == cudaSuccess ? 0 : -1;
}
static int tk_checks_get_here(int* out) {
    const int zero[2] = {0, 0};
    if (cudaMemcpyFromSymbol(out, tk_check_word_d, sizeof(zero)) != cudaSuccess) return -1;
    if (out[0] != 0) cudaMemcpyToSymbol(tk_check_word_d, zero, sizeof(zero));
    return 0;
}
namespace {
struct TkChecksRegistrar {
    TkChecksRegistrar() { tk_checks_register(tk_checks_set_here, tk_checks_get_here); }
};
static TkChecksRegistrar tk_checks_registrar;
}  // namespace

#else

#define TK_PAGE(kernel, page) (page)
#define TK_SLOT(kernel, slot) (slot)
#define TK_ROW(kernel, row, bound) (row)

#endif
