// Gated short convolution over a mixed batch, one kernel: u = round(B*X), causal depthwise
// conv of width W over u within each sequence, y = round(acc + bias), out = round(C*y), and the
// sequence's state row (its last W-1 values of u, newest last) replaced.
//
// Formulas: Tokenomos models/blocks/shortconv.py:39-59; kernels/conv/varlen.py:22-29,73-93,
// 134-145 (taps run from the oldest input to the current one, tap W-1 multiplies the current
// token; inputs before the sequence's first position are zero).
//
// A tile is a run of tokens of one sequence's portion; a thread owns one channel of one tile
// and walks its tokens in order with the last W-1 inputs in registers. Only the tile at offset
// 0 reads the state (its predecessors lie before the portion) and only that tile writes it,
// after it has read what it needs: every tile is at least W-1 tokens long (the last one of a
// portion excepted), so no other tile looks behind the portion. No second kernel, no race.
#include "common.cuh"

template <typename T, int W>
__global__ void conv_gated_kernel(const T* bcx, int64_t stride, int d,
                                  const float* __restrict__ w, const float* __restrict__ bias,
                                  T* state, T* out,
                                  const int* cu, const int* seq_ctx,
                                  const int* seq_slot,
                                  const int* tile_seq,
                                  const int* tile_off,
                                  const int* tile_n) {
    pdl_launch_dependents();
    pdl_wait();
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= d) return;
    const int s = tile_seq[blockIdx.x];
    const int off = tile_off[blockIdx.x];
    const int n = tile_n[blockIdx.x];
    const int start = cu[s];
    const int len = cu[s + 1] - start;
    const int ctx = seq_ctx[s];
    T* st = state + (size_t)seq_slot[s] * (W - 1) * d + c;

    float taps[W];
#pragma unroll
    for (int j = 0; j < W; ++j) taps[j] = w[(size_t)c * W + j];
    const float b = bias != nullptr ? bias[c] : 0.f;

    // u at index `li` of the portion (li may be negative: the state, or zero before position 0)
    auto input = [&](int li) -> float {
        if (li >= 0) {
            const T* row = bcx + (size_t)(start + li) * stride;
            return round_as<T>(to_f<T>(row[c]) * to_f<T>(row[2 * d + c]));
        }
        if (ctx + li < 0) return 0.f;
        return to_f<T>(st[(size_t)(W - 1 + li) * d]);
    };

    float hist[W - 1];
#pragma unroll
    for (int k = 0; k < W - 1; ++k) hist[k] = input(off - (W - 1) + k);

    float fresh[W - 1];
    const bool writes_state = off == 0;
    if (writes_state) {
        // the new state, read before anything of the old one is overwritten
#pragma unroll
        for (int k = 0; k < W - 1; ++k) fresh[k] = input(len - (W - 1) + k);
    }

    for (int i = 0; i < n; ++i) {
        const T* row = bcx + (size_t)(start + off + i) * stride;
        const float u = round_as<T>(to_f<T>(row[c]) * to_f<T>(row[2 * d + c]));
        float acc = 0.f;
#pragma unroll
        for (int j = 0; j < W - 1; ++j) acc += hist[j] * taps[j];
        acc += u * taps[W - 1];
        acc += b;
        const float y = round_as<T>(acc);
        out[(size_t)(start + off + i) * d + c] = from_f<T>(to_f<T>(row[d + c]) * y);
#pragma unroll
        for (int j = 0; j + 1 < W - 1; ++j) hist[j] = hist[j + 1];
        hist[W - 2] = u;
    }

    if (writes_state) {
#pragma unroll
        for (int k = 0; k < W - 1; ++k) st[(size_t)k * d] = from_f<T>(fresh[k]);
    }
}

template <typename T>
static int launch_conv(const void* bcx, int64_t stride, int d, const float* w, const float* bias,
                       void* state, void* out, const int* cu, const int* seq_ctx,
                       const int* seq_slot, const int* tile_seq, const int* tile_off,
                       const int* tile_n, int n_tiles, int W, cudaStream_t stream) {
    const int threads = 128;
    dim3 grid(n_tiles, (d + threads - 1) / threads);
#define TK_CONV_CASE(WW)                                                                         \
    case WW:                                                                                     \
        tk_launch(conv_gated_kernel<T, WW>, dim3(grid), dim3(threads), 0, stream,                                   \
            (const T*)bcx, stride, d, w, bias, (T*)state, (T*)out, cu, seq_ctx, seq_slot,        \
            tile_seq, tile_off, tile_n);                                                         \
        break;
    switch (W) {
        TK_CONV_CASE(2)
        TK_CONV_CASE(3)
        TK_CONV_CASE(4)
        TK_CONV_CASE(5)
        TK_CONV_CASE(6)
        TK_CONV_CASE(7)
        TK_CONV_CASE(8)
        default:
            tk_set_error("conv_gated: width %d outside 2..8", W);
            return -1;
    }
#undef TK_CONV_CASE
    TK_CHECK_LAUNCH("conv_gated");
    return 0;
}

// Smallest tile length (tokens) the caller may cut a portion into, for width W.
TK_API int tk_conv_min_tile(int W) { return W - 1; }

// bcx: [T, 3d] (B | C | X) with row stride `stride`; w: [d, W]; bias: [d] or null;
// state: [slots, W-1, d]; out: [T, d]; cu: [S+1]; seq_ctx, seq_slot: [S];
// tiles: sequence, offset in the sequence's portion, token count.
TK_API int tk_conv_gated(const void* bcx, int64_t stride, int d, const float* w, const float* bias,
                         void* state, void* out, const int* cu, const int* seq_ctx,
                         const int* seq_slot, const int* tile_seq, const int* tile_off,
                         const int* tile_n, int n_tiles, int W, int dtype, cudaStream_t stream) {
    TK_CHECK_ARG(d > 0 && n_tiles >= 0 && stride >= 3 * (int64_t)d, "conv_gated: bad sizes");
    if (n_tiles == 0) return 0;
    if (dtype == TK_F32)
        return launch_conv<float>(bcx, stride, d, w, bias, state, out, cu, seq_ctx, seq_slot,
                                  tile_seq, tile_off, tile_n, n_tiles, W, stream);
    if (dtype == TK_BF16)
        return launch_conv<__nv_bfloat16>(bcx, stride, d, w, bias, state, out, cu, seq_ctx,
                                          seq_slot, tile_seq, tile_off, tile_n, n_tiles, W, stream);
    TK_CHECK_ARG(false, "conv_gated: unknown dtype %d", dtype);
    return -1;
}
