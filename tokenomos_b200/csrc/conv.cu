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

// The form for prompt portions: a block of CONV_TT x CONV_CG threads takes tiles of up to CONV_TT
// tokens and CONV_CG groups of VEC channels, one thread per (token, group), `per_block` tiles of
// the list one after the other. A tile's rows (B, C and X of its tokens as stored, and the W - 1
// rows before it: rows of the portion, or the state with X = 1, or zeros) are copied into shared
// memory with cp.async, three tiles ahead of the one that is computed, and the tile list's
// entries are read a tile earlier still. A thread then sums its W taps over
// round(B * X) of its own and the W - 1 rows before, straight from the staged rows (16 bytes
// per thread and row, no bank conflicts), its taps in registers: one barrier per tile.
// (Earlier forms, a 2,048-token portion of 2,048 channels: a thread that walks 8 tokens 17 us;
// one tile per block through registers, u = B * X as 32-bit values in a second shared array
// 15.7 us, the same with this pipeline 16-17 us: the shared-memory pipe was two thirds busy, half
// of it bank conflicts of 32-byte rows, with two more barriers per tile.)
constexpr int CONV_MAX_W = 8;
constexpr int CONV_STAGES = 4;       // tiles whose rows are staged: one computed, three on their way

__device__ __forceinline__ void conv_cp16(void* dst, const void* src, bool valid) {
    const uint32_t d32 = (uint32_t)__cvta_generic_to_shared(dst);
    const int bytes = valid ? 16 : 0;                    // 0: sixteen zero bytes, nothing is read
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(d32), "l"(src), "r"(bytes));
}

// a tile's entry of the lists, and what only a portion's first tile needs beside it
struct ConvTile {
    int off, n, start, len, ctx, slot;
};

// INTER: a row of bcx holds (B, C, X) of 8 or 4 channels in turn (`block` == VEC, what the decode
// path's projection wants its rows as): a block's piece of a row is then one run of 3 CH values,
// copied as it lies and picked apart when read.
template <typename T, int W, int CONV_TT, int CONV_CG, bool INTER>
__global__ void __launch_bounds__(CONV_TT* CONV_CG, W <= 4 ? 3 : 2)
conv_gated_tile_kernel(const T* bcx, int64_t stride, int d, const float* __restrict__ w,
                       const float* __restrict__ bias, T* state, T* out, const int* cu,
                       const int* seq_ctx, const int* seq_slot, const int* tile_seq,
                       const int* tile_off, const int* tile_n, const int* tile_tok0, int block,
                       int n_tiles, int per_block) {
    constexpr int VEC = 16 / sizeof(T);
    constexpr int CH = CONV_CG * VEC;                         // channels of a block
    constexpr int HR = W - 1;                                 // rows before a tile
    extern __shared__ __align__(16) unsigned char conv_smem[];
    // [stage][B | X][HR + TT][CH] and [stage][C][TT][CH], as stored; INTER: [stage][HR + TT][3 CH]
    T* raw = reinterpret_cast<T*>(conv_smem);
    constexpr int STAGE = INTER ? 3 * (HR + CONV_TT) * CH : (2 * (HR + CONV_TT) + CONV_TT) * CH;
    // where this thread's B, X and C of staged row r lie, from the stage's start
    auto at_b = [&](int r) { return INTER ? r * 3 * CH + (int)threadIdx.x * 3 * VEC : r * CH + (int)threadIdx.x * VEC; };
    auto at_x = [&](int r) { return INTER ? at_b(r) + 2 * VEC : (HR + CONV_TT) * CH + at_b(r); };
    auto at_c = [&](int r) { return INTER ? at_b(r + HR) + VEC : 2 * (HR + CONV_TT) * CH + r * CH + (int)threadIdx.x * VEC; };
    __shared__ ConvTile entries[CONV_STAGES];                 // the staged tiles' entries
    pdl_launch_dependents();
    const int gi = threadIdx.x, ti = threadIdx.y;
    const int c0 = blockIdx.x * CH;     // channel blocks are the grid's fast axis: blocks that run
                                         // together read neighbouring pieces of the same rows
    const int c = c0 + gi * VEC;
    const bool live = c < d;
    // this thread's taps and bias (they do not depend on the kernel before this one)
    float taps[W][VEC], bias_r[VEC];
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
        bias_r[i] = live && bias != nullptr ? bias[c + i] : 0.f;
#pragma unroll
        for (int j = 0; j < W; ++j) taps[j][i] = live ? w[(size_t)(c + i) * W + j] : 0.f;
    }
    pdl_wait();
    const int first = blockIdx.y * per_block;
    const int count = min(per_block, n_tiles - first);
    const int cb = block ? (c / block) * 3 * block + c % block : c;
    const int cc = block ? cb + block : d + c, cx = block ? cb + 2 * block : 2 * d + c;

    auto read_entry = [&](int k) {
        ConvTile t;
        const int i = first + k;
        t.off = tile_off[i];
        t.n = tile_n[i];
        const int s = tile_seq[i];
        const int tok0 = tile_tok0 != nullptr ? tile_tok0[i] : -1;
        t.len = t.ctx = t.slot = 0;
        // a tile inside a portion needs nothing but its own entry; one at the portion's start
        // looks further: the sequence's length, cached count and slot
        if (t.n > 0 && t.off < HR) {
            t.start = cu[s];
            t.len = cu[s + 1] - t.start;
            t.ctx = seq_ctx[s];
            t.slot = TK_SLOT(TK_K_CONV, seq_slot[s]);
        } else {
            t.start = tok0 >= 0 ? tok0 - t.off : (t.n > 0 ? cu[s] : 0);
        }
        return t;
    };
    // the copies of one tile: its own rows, and by the first HR token rows the rows before it
    auto issue = [&](const ConvTile& t, int stage) {
        T* sg = raw + stage * STAGE;
        if (ti == 0 && gi == 0) entries[stage] = t;          // read back when the tile is computed
        if (t.n > 0) {
            const bool own = ti < t.n;
            const T* row = bcx + (size_t)(t.start + t.off + (own ? ti : 0)) * stride;
            const int li = t.off - HR + ti;               // of a row before the tile: its index in the portion
            const T* prev = bcx + (size_t)(t.start + (li >= 0 ? li : 0)) * stride;
            if constexpr (INTER) {
                // 3 CONV_CG pieces of 16 bytes per row, CONV_CG lanes: three pieces each
#pragma unroll
                for (int q = 0; q < 3; ++q) {
                    const int e = (gi + q * CONV_CG) * VEC;               // offset in the block's run
                    const bool inside = 3 * c0 + e < 3 * d;
                    conv_cp16(sg + (HR + ti) * 3 * CH + e, row + 3 * c0 + e, own && inside);
                    if (ti < HR && li >= 0) conv_cp16(sg + ti * 3 * CH + e, prev + 3 * c0 + e, inside);
                }
            } else if (live) {
                conv_cp16(sg + at_b(HR + ti), row + cb, own);
                conv_cp16(sg + at_x(HR + ti), row + cx, own);
                conv_cp16(sg + at_c(ti), row + cc, own);
                if (ti < HR && li >= 0) {
                    conv_cp16(sg + at_b(ti), prev + cb, true);
                    conv_cp16(sg + at_x(ti), prev + cx, true);
                }
            }
            if (live && ti < HR && li < 0) {
                // the state row (an input as it was stored), or zero before position 0; its
                // X is set to one when the copy has landed (`patch`)
                const bool held = t.ctx + li >= 0;
                const T* st_row = state + ((size_t)t.slot * HR + (held ? HR + li : 0)) * d + c;
                conv_cp16(sg + at_b(ti), st_row, held);
            }
        }
        asm volatile("cp.async.commit_group;\n" ::);
    };
    // a state row stands for B * X already: X = 1 makes the product the row itself (by the thread
    // that copied the row, after its copies have landed and before the barrier)
    auto patch = [&](const ConvTile& t, int stage) {
        if (t.n > 0 && live && ti < HR && t.off - HR + ti < 0) {
            T ones[VEC];
#pragma unroll
            for (int i = 0; i < VEC; ++i) ones[i] = from_f<T>(1.0f);
            *reinterpret_cast<uint4*>(raw + stage * STAGE + at_x(ti)) = *reinterpret_cast<const uint4*>(ones);
        }
    };

    if (count <= 0) return;
    // tiles 0 .. CONV_STAGES - 2 are asked for up front; every turn of the loop asks for one more
    // (with the entry that the turn before read) and reads the entry of the one after that
#pragma unroll
    for (int k = 0; k < CONV_STAGES - 1; ++k) {
        if (k < count) issue(read_entry(k), k);
        else asm volatile("cp.async.commit_group;\n" ::);
    }
    ConvTile ahead = read_entry(min(CONV_STAGES - 1, count - 1));
    __syncthreads();                // the first entries are in shared memory for everyone
    for (int k = 0; k < count; ++k) {
        const int stage = k % CONV_STAGES;
        asm volatile("cp.async.wait_group %0;\n" ::"n"(CONV_STAGES - 2));
        {
            // (the entry was stored at least one barrier ago)
            const ConvTile mine = entries[stage];
            patch(mine, stage);
        }
        __syncthreads();            // tile k has landed for every thread; tile k - 1 is computed
        const ConvTile t = entries[stage];
        const int want = k + CONV_STAGES - 1;
        if (want < count) issue(ahead, want % CONV_STAGES);      // into the stage tile k - 1 held
        else asm volatile("cp.async.commit_group;\n" ::);
        if (want + 1 < count) ahead = read_entry(want + 1);      // in flight while this tile is computed
        if (t.n <= 0) continue;     // an unused entry of a fixed-length list (captured steps)
        const T* sg = raw + stage * STAGE;
        const bool own = live && ti < t.n, halo = live && ti < HR;
        const bool writes_state = t.off == 0;
        // the portion's last inputs, for the state: asked for now, used after the sums
        uint4 fb = make_uint4(0u, 0u, 0u, 0u), fx = fb;
        bool f_product = false;
        T* st = state + (size_t)t.slot * HR * d + c;
        if (halo && writes_state) {
            const int li = t.len - HR + ti;
            if (li >= 0) {
                const T* row = bcx + (size_t)(t.start + li) * stride;
                fb = *reinterpret_cast<const uint4*>(row + cb);
                fx = *reinterpret_cast<const uint4*>(row + cx);
                f_product = true;
            } else if (t.ctx + li >= 0) {
                fb = *reinterpret_cast<const uint4*>(st + (size_t)(HR + li) * d);
            }
        }
        if (own) {
            float acc[VEC];
#pragma unroll
            for (int i = 0; i < VEC; ++i) acc[i] = 0.f;
#pragma unroll
            for (int j = 0; j < W; ++j) {
                const uint4 b_raw = *reinterpret_cast<const uint4*>(sg + at_b(ti + j));
                const uint4 x_raw = *reinterpret_cast<const uint4*>(sg + at_x(ti + j));
                if constexpr (sizeof(T) == 2) {
                    // the product of two bfloat16 values is exact in 32-bit, so the packed
                    // multiply's one rounding is round(B * X): a quarter of the instructions
                    const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&b_raw);
                    const __nv_bfloat162* x2 = reinterpret_cast<const __nv_bfloat162*>(&x_raw);
#pragma unroll
                    for (int i = 0; i < VEC / 2; ++i) {
                        const float2 u = __bfloat1622float2(__hmul2(b2[i], x2[i]));
                        acc[2 * i] += u.x * taps[j][2 * i];
                        acc[2 * i + 1] += u.y * taps[j][2 * i + 1];
                    }
                } else {
                    const T* bv = reinterpret_cast<const T*>(&b_raw);
                    const T* xv = reinterpret_cast<const T*>(&x_raw);
#pragma unroll
                    for (int i = 0; i < VEC; ++i) acc[i] += round_as<T>(to_f<T>(bv[i]) * to_f<T>(xv[i])) * taps[j][i];
                }
            }
            const uint4 rc = *reinterpret_cast<const uint4*>(sg + at_c(ti));
            const T* cv = reinterpret_cast<const T*>(&rc);
            uint4 packed;
            T* o = reinterpret_cast<T*>(&packed);
#pragma unroll
            for (int i = 0; i < VEC; ++i) {
                if (bias != nullptr) acc[i] += bias_r[i];
                o[i] = from_f<T>(to_f<T>(cv[i]) * round_as<T>(acc[i]));
            }
            *reinterpret_cast<uint4*>(out + (size_t)(t.start + t.off + ti) * d + c) = packed;
        }
        // The new state rows are the portion's last inputs; with a portion shorter than the
        // state some of them are old rows moved up, which every thread has read (above) before
        // any thread overwrites one (the barrier; `writes_state` is the same for the whole block).
        if (writes_state) __syncthreads();
        if (halo && writes_state) {
            const T* bv = reinterpret_cast<const T*>(&fb);
            const T* xv = reinterpret_cast<const T*>(&fx);
            uint4 packed;
            T* o = reinterpret_cast<T*>(&packed);
#pragma unroll
            for (int i = 0; i < VEC; ++i)
                o[i] = f_product ? from_f<T>(round_as<T>(to_f<T>(bv[i]) * to_f<T>(xv[i]))) : bv[i];
            *reinterpret_cast<uint4*>(st + (size_t)ti * d) = packed;
        }
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
    const int blocks_x = (d + cg * VEC - 1) / (cg * VEC);
    // tiles a block takes one after the other: as many blocks as are resident at once, the rest in a row
    const int resident = 148 * (W <= 4 ? 3 : 2);          // blocks the GPU holds at once (by registers)
    int tiles_each = (int)(((long long)blocks_x * n_tiles + resident - 1) / resident);
    tiles_each = tiles_each < 1 ? 1 : (tiles_each > 8 ? 8 : tiles_each);
    const dim3 tgrid(blocks_x, (n_tiles + tiles_each - 1) / tiles_each), tblock(cg, tt);
    const int ch = cg * VEC, hr = W - 1;
    const bool inter = block == VEC;
    const size_t tsmem = CONV_STAGES * (size_t)(inter ? 3 * (hr + tt) : 2 * (hr + tt) + tt) * ch * sizeof(T);
#define TK_CONV_TILED_I(WW, TT_, CG_, INTER_)                                                    \
    do {                                                                                         \
        static size_t allowed = 48 * 1024;      /* (one process drives one GPU) */               \
        if (tsmem > allowed) {                                                                   \
            cudaFuncSetAttribute(conv_gated_tile_kernel<T, WW, TT_, CG_, INTER_>,                \
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)tsmem);       \
            allowed = tsmem;                                                                     \
        }                                                                                        \
        tk_launch(conv_gated_tile_kernel<T, WW, TT_, CG_, INTER_>, tgrid, tblock, tsmem, stream, \
            (const T*)bcx, stride, d, w, bias, (T*)state, (T*)out, cu, seq_ctx, seq_slot,        \
            tile_seq, tile_off, tile_n, tile_tok0, block, n_tiles, tiles_each);                  \
    } while (0)
#define TK_CONV_TILED(WW, TT_, CG_)                                                              \
    do {                                                                                         \
        if (inter) TK_CONV_TILED_I(WW, TT_, CG_, true);                                          \
        else TK_CONV_TILED_I(WW, TT_, CG_, false);                                               \
    } while (0)
#define TK_CONV_CASE(WW)                                                                         \
    case WW:                                                                                     \
        if (tiled && tt == 16)                                                                   \
            TK_CONV_TILED(WW, 16, 16);                                                           \
        else if (tiled && tt == 8)                                                               \
            TK_CONV_TILED(WW, 8, 32);                                                            \
        else if (tiled && tt == 4 && WW <= 5)                                                    \
            TK_CONV_TILED(WW, (WW <= 5 ? 4 : 8), (WW <= 5 ? 64 : 32));                           \
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
#undef TK_CONV_TILED
#undef TK_CONV_TILED_I
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
