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
                                  const int* tile_n, int block) {
    pdl_launch_dependents();
    pdl_wait();
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= d) return;
    // columns of this channel's B, C and X in a row of bcx
    const int cb = block ? (c / block) * 3 * block + c % block : c;
    const int cc = block ? cb + block : d + c, cx = block ? cb + 2 * block : 2 * d + c;
    const int s = tile_seq[blockIdx.x];
    const int off = tile_off[blockIdx.x];
    const int n = tile_n[blockIdx.x];
    if (n <= 0) return;          // an unused entry of a fixed-length tile list (captured steps)
    const int start = cu[s];
    const int len = cu[s + 1] - start;
    const int ctx = seq_ctx[s];
    T* st = state + (size_t)TK_SLOT(TK_K_CONV, seq_slot[s]) * (W - 1) * d + c;

    float taps[W];
#pragma unroll
    for (int j = 0; j < W; ++j) taps[j] = w[(size_t)c * W + j];
    const float b = bias != nullptr ? bias[c] : 0.f;

    // u at index `li` of the portion (li may be negative: the state, or zero before position 0)
    auto input = [&](int li) -> float {
        if (li >= 0) {
            const T* row = bcx + (size_t)(start + li) * stride;
            return round_as<T>(to_f<T>(row[cb]) * to_f<T>(row[cx]));
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
        const float u = round_as<T>(to_f<T>(row[cb]) * to_f<T>(row[cx]));
        float acc = 0.f;
#pragma unroll
        for (int j = 0; j < W - 1; ++j) acc += hist[j] * taps[j];
        acc += u * taps[W - 1];
        acc += b;
        const float y = round_as<T>(acc);
        out[(size_t)(start + off + i) * d + c] = from_f<T>(to_f<T>(row[cc]) * y);
#pragma unroll
        for (int j = 0; j + 1 < W - 1; ++j) hist[j] = hist[j + 1];
        hist[W - 2] = u;
    }

    if (writes_state) {
#pragma unroll
        for (int k = 0; k < W - 1; ++k) st[(size_t)k * d] = from_f<T>(fresh[k]);
    }
}

// The same with 16-byte accesses: a thread owns VEC = 16 / sizeof(T) neighbouring channels of one
// tile, so every load and store moves whole 16-byte pieces of a token's row.
template <typename T, int W>
__global__ void conv_gated_vec_kernel(const T* bcx, int64_t stride, int d,
                                      const float* __restrict__ w, const float* __restrict__ bias,
                                      T* state, T* out, const int* cu, const int* seq_ctx,
                                      const int* seq_slot, const int* tile_seq, const int* tile_off,
                                      const int* tile_n, int block) {
    constexpr int VEC = 16 / sizeof(T);
    pdl_launch_dependents();
    pdl_wait();
    const int c = (blockIdx.y * blockDim.x + threadIdx.x) * VEC;
    if (c >= d) return;
    // columns of these channels' B, C and X in a row of bcx (a block is a multiple of VEC)
    const int cb = block ? (c / block) * 3 * block + c % block : c;
    const int cc = block ? cb + block : d + c, cx = block ? cb + 2 * block : 2 * d + c;
    const int s = tile_seq[blockIdx.x];
    const int off = tile_off[blockIdx.x];
    const int n = tile_n[blockIdx.x];
    if (n <= 0) return;          // an unused entry of a fixed-length tile list (captured steps)
    const int start = cu[s];
    const int len = cu[s + 1] - start;
    const int ctx = seq_ctx[s];
    T* st = state + (size_t)TK_SLOT(TK_K_CONV, seq_slot[s]) * (W - 1) * d + c;

    float taps[W][VEC], b[VEC];
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
#pragma unroll
        for (int j = 0; j < W; ++j) taps[j][i] = w[(size_t)(c + i) * W + j];
        b[i] = bias != nullptr ? bias[c + i] : 0.f;
    }
    auto load = [&](const T* p, float (&v)[VEC]) {
        const uint4 raw = *reinterpret_cast<const uint4*>(p);
        const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
        for (int i = 0; i < VEC; ++i) v[i] = to_f<T>(e[i]);
    };
    auto store = [&](T* p, const float (&v)[VEC]) {
        uint4 raw;
        T* e = reinterpret_cast<T*>(&raw);
#pragma unroll
        for (int i = 0; i < VEC; ++i) e[i] = from_f<T>(v[i]);
        *reinterpret_cast<uint4*>(p) = raw;
    };
    // u at index `li` of the portion (negative: the state, or zero before position 0)
    auto input = [&](int li, float (&u)[VEC]) {
        if (li >= 0) {
            const T* row = bcx + (size_t)(start + li) * stride;
            float bv[VEC], xv[VEC];
            load(row + cb, bv);
            load(row + cx, xv);
#pragma unroll
            for (int i = 0; i < VEC; ++i) u[i] = round_as<T>(bv[i] * xv[i]);
        } else if (ctx + li < 0) {
#pragma unroll
            for (int i = 0; i < VEC; ++i) u[i] = 0.f;
        } else {
            load(st + (size_t)(W - 1 + li) * d, u);
        }
    };

    float hist[W - 1][VEC];
#pragma unroll
    for (int k = 0; k < W - 1; ++k) input(off - (W - 1) + k, hist[k]);

    float fresh[W - 1][VEC];
    const bool writes_state = off == 0;
    if (writes_state) {
#pragma unroll
        for (int k = 0; k < W - 1; ++k) input(len - (W - 1) + k, fresh[k]);
    }

    // four tokens' loads are issued before the first of them is used
    for (int i0 = 0; i0 < n; i0 += 4) {
        uint4 rb[4], rc[4], rx[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            if (i0 + k < n) {
                const T* row = bcx + (size_t)(start + off + i0 + k) * stride;
                rb[k] = *reinterpret_cast<const uint4*>(row + cb);
                rc[k] = *reinterpret_cast<const uint4*>(row + cc);
                rx[k] = *reinterpret_cast<const uint4*>(row + cx);
            }
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            if (i0 + k >= n) break;
            const T* bv = reinterpret_cast<const T*>(&rb[k]);
            const T* cv = reinterpret_cast<const T*>(&rc[k]);
            const T* xv = reinterpret_cast<const T*>(&rx[k]);
            float y[VEC];
#pragma unroll
            for (int e = 0; e < VEC; ++e) {
                const float u = round_as<T>(to_f<T>(bv[e]) * to_f<T>(xv[e]));
                float acc = 0.f;
#pragma unroll
                for (int j = 0; j < W - 1; ++j) acc += hist[j][e] * taps[j][e];
                acc += u * taps[W - 1][e];
                acc += b[e];
                y[e] = to_f<T>(cv[e]) * round_as<T>(acc);
#pragma unroll
                for (int j = 0; j + 1 < W - 1; ++j) hist[j][e] = hist[j + 1][e];
                hist[W - 2][e] = u;
            }
            store(out + (size_t)(start + off + i0 + k) * d + c, y);
        }
    }

    if (writes_state) {
#pragma unroll
        for (int k = 0; k < W - 1; ++k) store(st + (size_t)k * d, fresh[k]);
    }
}

template <typename T>
static int launch_conv(const void* bcx, int64_t stride, int d, const float* w, const float* bias,
                       void* state, void* out, const int* cu, const int* seq_ctx,
                       const int* seq_slot, const int* tile_seq, const int* tile_off,
                       const int* tile_n, int n_tiles, int W, int block, cudaStream_t stream) {
    constexpr int VEC = 16 / sizeof(T);
    const bool vec_ok = d % VEC == 0 && block % VEC == 0 && stride % VEC == 0 && (uintptr_t)bcx % 16 == 0 && (uintptr_t)out % 16 == 0 &&
                        (uintptr_t)state % 16 == 0;
    const int threads = vec_ok ? 64 : 128;
    const int per_block = vec_ok ? threads * VEC : threads;
    dim3 grid(n_tiles, (d + per_block - 1) / per_block);
#define TK_CONV_CASE(WW)                                                                         \
    case WW:                                                                                     \
        if (vec_ok)                                                                              \
            tk_launch(conv_gated_vec_kernel<T, WW>, dim3(grid), dim3(threads), 0, stream,        \
                (const T*)bcx, stride, d, w, bias, (T*)state, (T*)out, cu, seq_ctx, seq_slot,    \
                tile_seq, tile_off, tile_n, block);                                              \
        else                                                                                     \
            tk_launch(conv_gated_kernel<T, WW>, dim3(grid), dim3(threads), 0, stream,            \
                (const T*)bcx, stride, d, w, bias, (T*)state, (T*)out, cu, seq_ctx, seq_slot,    \
                tile_seq, tile_off, tile_n, block);                                              \
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
// tiles: sequence, offset in the sequence's portion, token count. block 0: a row of bcx is all of
// B, then C, then X; block b > 0 (d a multiple of b): runs of b channels of B, of C and of X in turn.
TK_API int tk_conv_gated(const void* bcx, int64_t stride, int d, const float* w, const float* bias,
                         void* state, void* out, const int* cu, const int* seq_ctx,
                         const int* seq_slot, const int* tile_seq, const int* tile_off,
                         const int* tile_n, int n_tiles, int W, int block, int dtype, cudaStream_t stream) {
    TK_CHECK_ARG(d > 0 && n_tiles >= 0 && stride >= 3 * (int64_t)d, "conv_gated: bad sizes");
    TK_CHECK_ARG(block >= 0 && (block == 0 || d % block == 0), "conv_gated: %d channels in blocks of %d", d, block);
    if (n_tiles == 0) return 0;
    if (dtype == TK_F32)
        return launch_conv<float>(bcx, stride, d, w, bias, state, out, cu, seq_ctx, seq_slot,
                                  tile_seq, tile_off, tile_n, n_tiles, W, block, stream);
    if (dtype == TK_BF16)
        return launch_conv<__nv_bfloat16>(bcx, stride, d, w, bias, state, out, cu, seq_ctx,
                                          seq_slot, tile_seq, tile_off, tile_n, n_tiles, W, block, stream);
    TK_CHECK_ARG(false, "conv_gated: unknown dtype %d", dtype);
    return -1;
}
