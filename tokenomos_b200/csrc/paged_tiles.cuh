// Staging of paged keys and values in shared memory, shared by the attention kernels: 16-byte
// cp.async copies into [rows][D] bfloat16 tiles whose 16-byte chunks are XOR-swizzled by the row
// (for D = 64 this is exactly the 128-byte-swizzled K-major layout that ldmatrix reads without
// bank conflicts and that tcgen05.mma takes through a shared-memory descriptor).
#pragma once

#include "common.cuh"

namespace {

// 16 bytes global -> shared; `valid` false writes zeros instead (nothing is read)
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
    const int bytes = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

// byte offset of 16-byte chunk `chunk` of row `row` in a [rows][D] bf16 tile, XOR-swizzled so
// that the 8 rows an ldmatrix reads fall into different banks
template <int D>
__device__ __forceinline__ uint32_t tile_off(int row, int chunk) {
    return (uint32_t)(row * (D * 2) + ((chunk ^ (row & 7)) << 4));
}

// Load `rows` keys (or values) starting at key j0 of sequence `seq` into a swizzled tile with
// `nthreads` threads; keys outside [j_first, j_last] are zero-filled, not read.
template <int D>
__device__ __forceinline__ void load_tile(uint32_t tile, const __nv_bfloat16* pool,
                                          const int* bt_row, int j0, int rows,
                                          int j_first, int j_last, int kvh, int Hkv, int P, int which,
                                          int tid, int nthreads) {
    constexpr int CH = D / 8;
    for (int i = tid; i < rows * CH; i += nthreads) {
        const int r = i / CH, c = i % CH;
        const int j = j0 + r;
        const bool valid = j >= j_first && j <= j_last;
        const __nv_bfloat16* src = pool;
        if (valid) {
            const int page = TK_PAGE(TK_K_ATTN_TILES, bt_row[j / P]);
            src = pool + (((size_t)page * 2 + which) * Hkv + kvh) * (size_t)P * D +
                  (size_t)(j % P) * D + c * 8;
        }
        cp_async16(tile + tile_off<D>(r, c), src, valid);
    }
}

// The same load for page sizes that are a power of two, which is what the engine uses: a thread
// owns one 16-byte column of ROWS / (NT / CH) rows of every tile, so everything but the page
// lookup is computed once per kernel instead of once per 16 bytes. Keys and values of a row share
// the lookup (the value row lies a constant distance behind the key row).
template <int D, int ROWS, int NT>
struct PagedLoader {
    static constexpr int CH = D / 8;
    static constexpr int STEP = NT / CH;          // rows between a thread's consecutive rows
    static constexpr int PER = ROWS / STEP;       // rows per thread per tile
    uint32_t dst[PER];                            // swizzled byte offsets inside a tile
    int r0;
    size_t head_off, v_delta, page_stride;
    int p_shift, p_mask;

    __device__ __forceinline__ void init(int tid, int kvh, int Hkv, int P, int shift) {
        const int c = tid % CH;
        r0 = tid / CH;
#pragma unroll
        for (int k = 0; k < PER; ++k) dst[k] = tile_off<D>(r0 + k * STEP, c);
        head_off = (size_t)kvh * P * D + (size_t)c * 8;
        v_delta = (size_t)Hkv * P * D;
        page_stride = (size_t)2 * Hkv * P * D;
        p_shift = shift;
        p_mask = P - 1;
    }

    __device__ __forceinline__ void issue(uint32_t ktile, uint32_t vtile, const __nv_bfloat16* pool,
                                          const int* bt_row, int j0, int j_first, int j_last) const {
#pragma unroll
        for (int k = 0; k < PER; ++k) {
            const int j = j0 + r0 + k * STEP;
            const bool valid = j >= j_first && j <= j_last;
            const __nv_bfloat16* src = pool;
            if (valid) {
                const int page = TK_PAGE(TK_K_ATTN_TILES, bt_row[j >> p_shift]);
                src = pool + (size_t)page * page_stride + head_off + (size_t)(j & p_mask) * D;
            }
            cp_async16(ktile + dst[k], src, valid);
            cp_async16(vtile + dst[k], valid ? src + v_delta : src, valid);
        }
    }

    // The same in two halves, so that the block-table loads of a tile are in flight long before
    // its copies are issued (four dependent lookups in a row otherwise sit on the loader's path):
    // lookup() fetches the page numbers of the tile at j0, issue_looked_up() uses them.
    int page[PER];

    __device__ __forceinline__ void lookup(const int* bt_row, int j0, int j_first, int j_last) {
#pragma unroll
        for (int k = 0; k < PER; ++k) {
            const int j = min(max(j0 + r0 + k * STEP, j_first), j_last);     // always a held position
            page[k] = TK_PAGE(TK_K_ATTN_TILES, bt_row[j >> p_shift]);
        }
    }

    __device__ __forceinline__ void issue_looked_up(uint32_t ktile, uint32_t vtile, const __nv_bfloat16* pool,
                                                    int j0, int j_first, int j_last) const {
#pragma unroll
        for (int k = 0; k < PER; ++k) {
            const int j = j0 + r0 + k * STEP;
            const bool valid = j >= j_first && j <= j_last;
            const __nv_bfloat16* src = pool;
            if (valid) src = pool + (size_t)page[k] * page_stride + head_off + (size_t)(j & p_mask) * D;
            cp_async16(ktile + dst[k], src, valid);
            cp_async16(vtile + dst[k], valid ? src + v_delta : src, valid);
        }
    }
};

constexpr float LOG2E = 1.4426950408889634f;

// 2^x on the special-function unit (about 2 ulp in 32-bit, far below the bfloat16 rounding of P);
// -inf gives 0, which the masking relies on
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

}  // namespace
