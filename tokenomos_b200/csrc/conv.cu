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
    // Every load of a thread's first four tokens, of the W - 1 inputs before them and (in the
    // tile that owns the state) of the portion's last W - 1 inputs is issued before any is used:
    // one trip to memory for a tile of up to four tokens instead of three, one behind the other.
    // An input at index li of the portion is B * X of that row, or, before the portion, the
    // state row (zero before position 0).
    // (the portion's last inputs only for widths up to 4: wider ones would spill registers, and
    // fetch them after the loop instead)
    constexpr bool EARLY = W <= 4;
    const bool writes_state = off == 0;
    const uint4 zero4 = make_uint4(0u, 0u, 0u, 0u);
    uint4 hb[W - 1], hx[W - 1], fb[EARLY ? W - 1 : 1], fx[EARLY ? W - 1 : 1];
    auto fetch_fresh = [&](int k, uint4& b_raw, uint4& x_raw) {
        b_raw = x_raw = zero4;
        const int lf = len - (W - 1) + k;
        if (lf >= 0) {
            const T* row = bcx + (size_t)(start + lf) * stride;
            b_raw = *reinterpret_cast<const uint4*>(row + cb);
            x_raw = *reinterpret_cast<const uint4*>(row + cx);
        } else if (ctx + lf >= 0) {
            b_raw = *reinterpret_cast<const uint4*>(st + (size_t)(W - 1 + lf) * d);
        }
    };
#pragma unroll
    for (int k = 0; k < W - 1; ++k) {
        const int li = off - (W - 1) + k;
        if (li >= 0) {
            const T* row = bcx + (size_t)(start + li) * stride;
            hb[k] = *reinterpret_cast<const uint4*>(row + cb);
            hx[k] = *reinterpret_cast<const uint4*>(row + cx);
        } else {
            hb[k] = ctx + li < 0 ? zero4 : *reinterpret_cast<const uint4*>(st + (size_t)(W - 1 + li) * d);
            hx[k] = zero4;
        }
        if constexpr (EARLY) {
            fb[k] = fx[k] = zero4;
            if (writes_state) fetch_fresh(k, fb[k], fx[k]);
        }
    }
    uint4 rb[4], rc[4], rx[4];
    auto fetch = [&](int i0) {
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            if (i0 + k < n) {
                const T* row = bcx + (size_t)(start + off + i0 + k) * stride;
                rb[k] = *reinterpret_cast<const uint4*>(row + cb);
                rc[k] = *reinterpret_cast<const uint4*>(row + cc);
                rx[k] = *reinterpret_cast<const uint4*>(row + cx);
            }
        }
    };
    fetch(0);
    // a raw pair (B, X) of a row of the batch, or a raw state row, as the input it stands for
    auto as_input = [&](int li, const uint4& b_raw, const uint4& x_raw, float (&u)[VEC]) {
        const T* bv = reinterpret_cast<const T*>(&b_raw);
        const T* xv = reinterpret_cast<const T*>(&x_raw);
#pragma unroll
        for (int i = 0; i < VEC; ++i)
            u[i] = li >= 0 ? round_as<T>(to_f<T>(bv[i]) * to_f<T>(xv[i])) : to_f<T>(bv[i]);
    };
    float hist[W - 1][VEC], fresh[EARLY ? W - 1 : 1][VEC];
#pragma unroll
    for (int k = 0; k < W - 1; ++k) {
        as_input(off - (W - 1) + k, hb[k], hx[k], hist[k]);
        if constexpr (EARLY) as_input(len - (W - 1) + k, fb[k], fx[k], fresh[k]);
    }

    for (int i0 = 0; i0 < n; i0 += 4) {
        if (i0 > 0) fetch(i0);
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
        if constexpr (EARLY) {
#pragma unroll
            for (int k = 0; k < W - 1; ++k) store(st + (size_t)k * d, fresh[k]);
        } else {
            // every new row is read before the first old one is overwritten
            uint4 lb[W - 1], lx[W - 1];
#pragma unroll
            for (int k = 0; k < W - 1; ++k) fetch_fresh(k, lb[k], lx[k]);
#pragma unroll
            for (int k = 0; k < W - 1; ++k) {
                float u[VEC];
                as_input(len - (W - 1) + k, lb[k], lx[k], u);
                store(st + (size_t)k * d, u);
            }
        }
    }
}

// The form for prompt portions: a block takes a tile of up to CONV_TT tokens and CONV_CG groups
// of VEC channels, one thread per (token, group). Every thread loads its own row's B, C and X
// (16 bytes each), the first W - 1 token rows of the block also load the W - 1 inputs before the
// tile (rows of the portion, or the state), u = B * X goes to shared memory, and after one
// barrier every thread sums its W taps over shared memory. Few registers, every load of the
// block in flight at once: the kernel runs at memory speed where the walking form above is bound
// by the latency of its dependent trips (a 2,048-token portion of 2,048 channels: 17 us there).
constexpr int CONV_MAX_W = 8;

template <typename T, int W, int CONV_TT, int CONV_CG>
__global__ void __launch_bounds__(CONV_TT* CONV_CG)
conv_gated_tile_kernel(const T* bcx, int64_t stride, int d, const float* __restrict__ w,
                       const float* __restrict__ bias, T* state, T* out, const int* cu,
                       const int* seq_ctx, const int* seq_slot, const int* tile_seq,
                       const int* tile_off, const int* tile_n, const int* tile_tok0, int block) {
    constexpr int VEC = 16 / sizeof(T);
    constexpr int CH = CONV_CG * VEC;                         // channels of a block
    __shared__ __align__(16) float u_s[CONV_TT + W - 1][CH];
    __shared__ __align__(16) float taps_s[W][CH];
    pdl_launch_dependents();
    const int gi = threadIdx.x, ti = threadIdx.y;
    const int c0 = blockIdx.x * CH;     // channel blocks are the grid's fast axis: blocks that run
                                         // together read neighbouring pieces of the same rows
    const int c = c0 + gi * VEC;
    const bool live = c < d;
    // the taps do not depend on the kernel before this one
    for (int i = ti * CONV_CG + gi; i < CH * W; i += CONV_TT * CONV_CG) {
        const int ch = i / W, j = i % W;
        taps_s[j][ch] = c0 + ch < d ? w[(size_t)(c0 + ch) * W + j] : 0.f;
    }
    pdl_wait();
    // Trips to memory, one behind the other, are what a block's time is made of. A tile inside a
    // portion (off >= W - 1) needs one for its entry of the tile lists and one for its rows; only
    // a tile at the portion's start looks further: the sequence's length, cached count and slot.
    const int off = tile_off[blockIdx.y];
    const int n = tile_n[blockIdx.y];
    const int s = tile_seq[blockIdx.y];
    const int tok0 = tile_tok0 != nullptr ? tile_tok0[blockIdx.y] : -1;
    if (n <= 0) return;          // an unused entry of a fixed-length tile list (captured steps)
    const bool at_start = off < W - 1;
    const int start = (tok0 >= 0 && !at_start) ? tok0 - off : cu[s];
    int len = 0, ctx = 0;
    T* st = state + c;
    if (at_start) {
        len = cu[s + 1] - start;
        ctx = seq_ctx[s];
        st += (size_t)TK_SLOT(TK_K_CONV, seq_slot[s]) * (W - 1) * d;
    }
    const int cb = block ? (c / block) * 3 * block + c % block : c;
    const int cc = block ? cb + block : d + c, cx = block ? cb + 2 * block : 2 * d + c;
    const uint4 zero4 = make_uint4(0u, 0u, 0u, 0u);
    const bool writes_state = off == 0;

    // an input at index li of the portion, as raw 16-byte pieces: (B, X) of that row, or the
    // state row (in `b_raw`) before the portion, or zero before position 0
    auto fetch = [&](int li, uint4& b_raw, uint4& x_raw) {
        b_raw = x_raw = zero4;
        if (li >= 0) {
            const T* row = bcx + (size_t)(start + li) * stride;
            b_raw = *reinterpret_cast<const uint4*>(row + cb);
            x_raw = *reinterpret_cast<const uint4*>(row + cx);
        } else if (ctx + li >= 0) {
            b_raw = *reinterpret_cast<const uint4*>(st + (size_t)(W - 1 + li) * d);
        }
    };
    auto as_input = [&](int li, const uint4& b_raw, const uint4& x_raw, float (&u)[VEC]) {
        const T* bv = reinterpret_cast<const T*>(&b_raw);
        const T* xv = reinterpret_cast<const T*>(&x_raw);
#pragma unroll
        for (int i = 0; i < VEC; ++i)
            u[i] = li >= 0 ? round_as<T>(to_f<T>(bv[i]) * to_f<T>(xv[i])) : to_f<T>(bv[i]);
    };

    uint4 rb = zero4, rx = zero4, rc = zero4, hb = zero4, hx = zero4, fb = zero4, fx = zero4;
    const bool own = live && ti < n, halo = live && ti < W - 1;
    if (own) {
        const T* row = bcx + (size_t)(start + off + ti) * stride;
        rb = *reinterpret_cast<const uint4*>(row + cb);
        rx = *reinterpret_cast<const uint4*>(row + cx);
        rc = *reinterpret_cast<const uint4*>(row + cc);
    }
    if (halo) {
        fetch(off - (W - 1) + ti, hb, hx);
        if (writes_state) fetch(len - (W - 1) + ti, fb, fx);
    }
    // shared memory is written and read four floats at a time
    auto put = [&](float* dst, const float (&v)[VEC]) {
#pragma unroll
        for (int i = 0; i < VEC; i += 4) *reinterpret_cast<float4*>(dst + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
    };
    auto get = [&](const float* src, float (&v)[VEC]) {
#pragma unroll
        for (int i = 0; i < VEC; i += 4) {
            const float4 f = *reinterpret_cast<const float4*>(src + i);
            v[i] = f.x, v[i + 1] = f.y, v[i + 2] = f.z, v[i + 3] = f.w;
        }
    };
    float u[VEC];
    if (own) {
        as_input(0, rb, rx, u);
        put(&u_s[W - 1 + ti][gi * VEC], u);
    }
    if (halo) {
        as_input(off - (W - 1) + ti, hb, hx, u);
        put(&u_s[ti][gi * VEC], u);
    }
    __syncthreads();
    if (own) {
        float acc[VEC], in[VEC], tp[VEC];
#pragma unroll
        for (int i = 0; i < VEC; ++i) acc[i] = 0.f;
#pragma unroll
        for (int j = 0; j < W; ++j) {
            get(&u_s[ti + j][gi * VEC], in);
            get(&taps_s[j][gi * VEC], tp);
#pragma unroll
            for (int i = 0; i < VEC; ++i) acc[i] += in[i] * tp[i];
        }
        const T* cv = reinterpret_cast<const T*>(&rc);
        uint4 packed;
        T* o = reinterpret_cast<T*>(&packed);
#pragma unroll
        for (int i = 0; i < VEC; ++i) {
            if (bias != nullptr) acc[i] += bias[c + i];
            o[i] = from_f<T>(to_f<T>(cv[i]) * round_as<T>(acc[i]));
        }
        *reinterpret_cast<uint4*>(out + (size_t)(start + off + ti) * d + c) = packed;
    }
    if (halo && writes_state) {
        // the old rows were read before the barrier; the new ones are the portion's last inputs
        as_input(len - (W - 1) + ti, fb, fx, u);
        uint4 packed;
        T* o = reinterpret_cast<T*>(&packed);
#pragma unroll
        for (int i = 0; i < VEC; ++i) o[i] = from_f<T>(u[i]);
        *reinterpret_cast<uint4*>(st + (size_t)ti * d) = packed;
    }
}

template <typename T>
static int launch_conv(const void* bcx, int64_t stride, int d, const float* w, const float* bias,
                       void* state, void* out, const int* cu, const int* seq_ctx,
                       const int* seq_slot, const int* tile_seq, const int* tile_off,
                       const int* tile_n, const int* tile_tok0, int n_tiles, int W, int block, int tile_cap,
                       cudaStream_t stream) {
    constexpr int VEC = 16 / sizeof(T);
    const bool vec_ok = d % VEC == 0 && block % VEC == 0 && stride % VEC == 0 && (uintptr_t)bcx % 16 == 0 && (uintptr_t)out % 16 == 0 &&
                        (uintptr_t)state % 16 == 0;
    const int threads = vec_ok ? 64 : 128;
    const int per_block = vec_ok ? threads * VEC : threads;
    dim3 grid(n_tiles, (d + per_block - 1) / per_block);
    // tiles of at most 16 tokens (and at least W - 1, as every form needs): the tiled form, a
    // block of 256 threads shaped to the tile (16 x 16 groups of channels, 8 x 32 or 4 x 64)
    const bool tiled = vec_ok && tile_cap >= W - 1 && tile_cap >= 1 && tile_cap <= 16 && W <= CONV_MAX_W &&
                       n_tiles <= 65535;
    const int tt = tile_cap <= 4 ? 4 : (tile_cap <= 8 ? 8 : 16), cg = 256 / tt;
    const dim3 tgrid((d + cg * VEC - 1) / (cg * VEC), n_tiles), tblock(cg, tt);
#define TK_CONV_CASE(WW)                                                                         \
    case WW:                                                                                     \
        if (tiled && tt == 16)                                                                   \
            tk_launch(conv_gated_tile_kernel<T, WW, 16, 16>, tgrid, tblock, 0, stream,           \
                (const T*)bcx, stride, d, w, bias, (T*)state, (T*)out, cu, seq_ctx, seq_slot,    \
                tile_seq, tile_off, tile_n, tile_tok0, block);                                   \
        else if (tiled && tt == 8 && WW <= 9)                                                    \
            tk_launch(conv_gated_tile_kernel<T, WW, 8, 32>, tgrid, tblock, 0, stream,            \
                (const T*)bcx, stride, d, w, bias, (T*)state, (T*)out, cu, seq_ctx, seq_slot,    \
                tile_seq, tile_off, tile_n, tile_tok0, block);                                   \
        else if (tiled && tt == 4 && WW <= 5)                                                    \
            tk_launch(conv_gated_tile_kernel<T, WW, (WW <= 5 ? 4 : 8), (WW <= 5 ? 64 : 32)>, tgrid, tblock, 0, stream, \
                (const T*)bcx, stride, d, w, bias, (T*)state, (T*)out, cu, seq_ctx, seq_slot,    \
                tile_seq, tile_off, tile_n, tile_tok0, block);                                   \
        else if (vec_ok)                                                                         \
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
// tile_cap: the most tokens a tile has (0: unknown); up to 16 the tiled kernel takes the call.
// tile_tok0 (optional): each tile's first token in the batch (= cu[seq] + offset), which spares
// the tiled kernel a dependent lookup.
TK_API int tk_conv_gated(const void* bcx, int64_t stride, int d, const float* w, const float* bias,
                         void* state, void* out, const int* cu, const int* seq_ctx,
                         const int* seq_slot, const int* tile_seq, const int* tile_off,
                         const int* tile_n, const int* tile_tok0, int n_tiles, int W, int block,
                         int tile_cap, int dtype, cudaStream_t stream) {
    TK_CHECK_ARG(d > 0 && n_tiles >= 0 && stride >= 3 * (int64_t)d, "conv_gated: bad sizes");
    TK_CHECK_ARG(block >= 0 && (block == 0 || d % block == 0), "conv_gated: %d channels in blocks of %d", d, block);
    if (n_tiles == 0) return 0;
    if (dtype == TK_F32)
        return launch_conv<float>(bcx, stride, d, w, bias, state, out, cu, seq_ctx, seq_slot,
                                  tile_seq, tile_off, tile_n, tile_tok0, n_tiles, W, block, tile_cap, stream);
    if (dtype == TK_BF16)
        return launch_conv<__nv_bfloat16>(bcx, stride, d, w, bias, state, out, cu, seq_ctx,
                                          seq_slot, tile_seq, tile_off, tile_n, tile_tok0, n_tiles, W, block, tile_cap, stream);
    TK_CHECK_ARG(false, "conv_gated: unknown dtype %d", dtype);
    return -1;
}
