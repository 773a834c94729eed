/* Entry points of libtokenomos_b200 that allocate nothing.
 *
 * This header has no counterpart in the reference (KohakuBlueleaf/Tokenomos launches its
 * kernels from Python with tensors its allocator made). It is for users of this library who
 * call it from a place where no device memory can be requested: inside a stream capture that
 * belongs to someone else, from a serving loop whose memory pool is spoken for, or through a
 * plain C binding that has no allocator to offer.
 *
 * tk_attn_decode_mma_static is tk_attn_decode_mma (split decode attention over the paged
 * cache, bfloat16, head size 64 or 128) with one difference: the scratch that holds the
 * per-split partial results is an array inside the library image instead of a buffer from the
 * caller. The caller still passes every input and the output.
 *
 *   - Limit: n * H * nsplit * (D + 2) floats must fit the array,
 *     tk_attn_decode_mma_static_capacity() floats (2 Mi floats, 8 MiB). Larger requests are
 *     refused with a message; nothing is launched. Every GPU that loads the library holds the
 *     array until the process exits.
 *   - The first call on a device looks up the array's device address (cudaGetSymbolAddress,
 *     with that device current). Make that first call before any stream capture begins.
 *     Host threads: any thread may make it; if two threads make the first call on one device
 *     at the same moment, both look the address up and store the same value, which is
 *     harmless. After it, the entry point reads that value and nothing else of its own.
 *   - It calls no cudaMalloc, cudaFree or allocating library routine.
 *   - All calls share the one array, and it keeps what the last call left. Nothing in it needs
 *     to start at zero: every slot a call reads was written by that call's own first kernel.
 *     Two calls that overlap on the GPU (issued on different streams without an event between
 *     them) would write the same slots and race: keep them in one stream, or order them.
 *   - Returns 0, or a negative code with the message in tk_last_error().
 */
#pragma once

#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

long long tk_attn_decode_mma_static_capacity(void);

int tk_attn_decode_mma_static(const void* q, const void* kv_pool, void* out, const int* positions,
                              const int* tok_seq, const int* block_table, int bt_stride,
                              const int* tok_index, int n, int H, int Hkv, int D, int P, int window,
                              float scale, int nsplit, cudaStream_t stream);

const char* tk_last_error(void);

#ifdef __cplusplus
}
#endif
