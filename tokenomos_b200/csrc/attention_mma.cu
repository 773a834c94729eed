// Paged attention on the tensor cores for bfloat16 and head sizes 64 and 128 (warp-level
// mma.sync m16n8k16, cp.async staging, online softmax in 32-bit).
//
// Rows of a tile are (token, query head) pairs that share one KV head, so the group's heads
// reuse every key and value that is loaded.
//   prefill kernel: a CTA takes up to 64 rows (64/G tokens of one sequence, G heads each), four
//     warps of 16 rows, and walks the keys in tiles of 64 through a double-buffered cp.async
//     pipeline; keys come from the paged cache, this step's own keys included.
//   decode kernel: one token per sequence, its G heads are the (padded) 16 rows; the four warps
//     of a CTA take alternate 32-key tiles of the CTA's key range, and `nsplit` CTAs split one
//     sequence's keys so that small batches still fill the GPU. Partial results (row maximum,
//     row sum, unnormalised output) go to scratch memory and a second kernel merges them.
//   fused decode kernel (steps of a few single tokens): the same walk with the q/k norm, the
//     rotation, the cache write, the merge (by the last CTA to finish) and the head gate in it.
// The kernels apply the per-head output gate as they write, when the layer has one.
// Masking, scale, rounding of P to bfloat16 and the unrounded row sum follow the generic kernel
// (Tokenomos kernels/attention/paged.py:67-76,150,267; models/blocks/attention.py:31-40,173).
// Keys past a query's position are never read: their shared-memory rows are zero-filled.
#include "no_alloc.h"
#include <math.h>

#include "paged_tiles.cuh"

namespace {

__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0,
                                         uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
        "{%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}

__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}

// The per-head output gate of (token, head): round(sigmoid(g)), or 1 without a gate. A gated
// output element is round(round(o) * gate), as the separate gate kernel computes it.
__device__ __forceinline__ float head_gate_of(const __nv_bfloat16* gate, int64_t ldg, int tok, int head) {
    if (gate == nullptr) return 1.0f;
    const float g = __bfloat162float(gate[(size_t)tok * ldg + head]);
    return round_as<__nv_bfloat16>(1.0f / (1.0f + expf(-g)));
}

// One 16-row x NK-key block of the online softmax for a warp: S = Q K^T from `ktile`, mask,
// update (m, l, O) with V from `vtile`. NK is 64 (prefill) or 32 (decode).
template <int D, int NK>
__device__ __forceinline__ void warp_block(const uint32_t (&qf)[D / 16][4], uint32_t ktile,
                                           uint32_t vtile, int j0, int pos_lo, int pos_hi,
                                           int window, float scale_log2, bool need_mask,
                                           float (&m)[2], float (&l)[2], float (&o)[D / 8][4]) {
    const int lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    float s[NK / 8][4];
#pragma unroll
    for (int n = 0; n < NK / 8; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) s[n][e] = 0.f;
    // S = Q K^T: for each pair of 8-key tiles and each 16-wide slice of the head
    {
        const int mi = lane >> 3, r = lane & 7;
#pragma unroll
        for (int np = 0; np < NK / 16; ++np) {
            const int key = np * 16 + r + 8 * (mi >> 1);
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks) {
                uint32_t b[4];
                ldmatrix_x4(b, ktile + tile_off<D>(key, ks * 2 + (mi & 1)));
                mma16816(s[2 * np], qf[ks], b[0], b[1]);
                mma16816(s[2 * np + 1], qf[ks], b[2], b[3]);
            }
        }
    }
    // mask: rows g (position pos_lo) and g + 8 (position pos_hi); key of element e of tile n
    if (need_mask) {
#pragma unroll
        for (int n = 0; n < NK / 8; ++n) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int j = j0 + n * 8 + 2 * t + (e & 1);
                const int pos = (e < 2) ? pos_lo : pos_hi;
                const bool visible = j <= pos && (window <= 0 || pos - j < window);
                if (!visible) s[n][e] = -INFINITY;
            }
        }
    }
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int n = 0; n < NK / 8; ++n) {
        mx[0] = fmaxf(mx[0], fmaxf(s[n][0], s[n][1]));
        mx[1] = fmaxf(mx[1], fmaxf(s[n][2], s[n][3]));
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
        mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
    }
    float alpha[2], msafe[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const float m_new = fmaxf(m[h], mx[h]);
        msafe[h] = m_new == -INFINITY ? 0.f : m_new;
        alpha[h] = fast_exp2((m[h] - msafe[h]) * scale_log2);
        m[h] = m_new;
        l[h] *= alpha[h];
    }
    uint32_t pf[NK / 16][4];
#pragma unroll
    for (int n = 0; n < NK / 8; ++n) {
        const float p0 = fast_exp2((s[n][0] - msafe[0]) * scale_log2);
        const float p1 = fast_exp2((s[n][1] - msafe[0]) * scale_log2);
        const float p2 = fast_exp2((s[n][2] - msafe[1]) * scale_log2);
        const float p3 = fast_exp2((s[n][3] - msafe[1]) * scale_log2);
        l[0] += p0 + p1;
        l[1] += p2 + p3;
        // the C layout of two neighbouring 8-key tiles is the A layout of one 16-key step
        pf[n >> 1][(n & 1) * 2 + 0] = pack_bf16(p0, p1);
        pf[n >> 1][(n & 1) * 2 + 1] = pack_bf16(p2, p3);
    }
#pragma unroll
    for (int n = 0; n < D / 8; ++n) {
        o[n][0] *= alpha[0];
        o[n][1] *= alpha[0];
        o[n][2] *= alpha[1];
        o[n][3] *= alpha[1];
    }
    // O += P V
    {
        const int mi = lane >> 3, r = lane & 7;
#pragma unroll
        for (int ks = 0; ks < NK / 16; ++ks) {
            const int key = ks * 16 + r + 8 * (mi & 1);
#pragma unroll
            for (int dp = 0; dp < D / 16; ++dp) {
                uint32_t b[4];
                ldmatrix_x4_trans(b, vtile + tile_off<D>(key, dp * 2 + (mi >> 1)));
                mma16816(o[2 * dp], pf[ks], b[0], b[1]);
                mma16816(o[2 * dp + 1], pf[ks], b[2], b[3]);
            }
        }
    }
}

// Query fragments of 16 rows straight from global memory. Row r of the warp is
// (token tok0 + r / G, head h0 + r % G); rows at or past `rows` read as zero.
template <int D>
__device__ __forceinline__ void load_q(uint32_t (&qf)[D / 16][4], const __nv_bfloat16* q,
                                       int row0, int rows, int tok0, int G, int H, int h0) {
    const int lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int r = row0 + g + 8 * half;
        const bool ok = r < rows;
        const __nv_bfloat16* src = q;
        const int gs = 31 - __clz(G);                 // the group size is a power of two
        if (ok) src = q + ((size_t)(tok0 + (r >> gs)) * H + h0 + (r & (G - 1))) * D;
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
            uint32_t lo = 0u, hi = 0u;
            if (ok) {
                lo = *reinterpret_cast<const uint32_t*>(src + ks * 16 + 2 * t);
                hi = *reinterpret_cast<const uint32_t*>(src + ks * 16 + 8 + 2 * t);
            }
            qf[ks][half] = lo;       // a0 (row g) / a1 (row g + 8): columns 2t, 2t + 1
            qf[ks][half + 2] = hi;   // a2 / a3: columns 2t + 8, 2t + 9
        }
    }
}

// ---------------------------------------------------------------------------------------------
// prefill: 64 rows per CTA, all keys
// ---------------------------------------------------------------------------------------------
template <int D>
__global__ void __launch_bounds__(128, (D == 64 ? 4 : 2))
attn_prefill_mma_kernel(const __nv_bfloat16* q, const __nv_bfloat16* pool,
                        __nv_bfloat16* out, const int* positions,
                        const int* tok_seq, const int* block_table,
                        int bt_stride, const int* tile_tok0,
                        const int* tile_ntok, int H, int Hkv, int P, int window,
                        float scale, int p_shift, const __nv_bfloat16* gate, int64_t ldg) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ __align__(128) unsigned char smem_raw[];
    constexpr int TILE_BYTES = 64 * D * 2;
    const uint32_t smem = smem_u32(smem_raw);   // [stage][K|V][64][D]
    const int G = H / Hkv;
    // the grid is one-dimensional with the KV head fastest and the tiles in reverse: a causal
    // tile late in its sequence reads the most keys, so the longest CTAs start first and the
    // last wave is made of short ones
    const int kvh = blockIdx.x % Hkv;
    const int tile = gridDim.x / Hkv - 1 - blockIdx.x / Hkv;
    const int tok0 = tile_tok0[tile], ntok = tile_ntok[tile];
    if (ntok <= 0) return;       // an unused entry of a fixed-length tile list (captured steps)
    const int rows = ntok * G;
    const int seq = tok_seq[tok0];
    const int* bt_row = block_table + (size_t)seq * bt_stride;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2;
    const int pos_first = positions[tok0];
    const int pos_last = pos_first + ntok - 1;       // consecutive positions within a tile
    const int lo = window > 0 ? max(0, pos_first - window + 1) : 0;
    const int j_begin = (lo / 64) * 64;

    uint32_t qf[D / 16][4];
    load_q<D>(qf, q, warp * 16, rows, tok0, G, H, kvh * G);
    const int r_lo = warp * 16 + g, r_hi = r_lo + 8;
    const int pos_lo = r_lo < rows ? pos_first + r_lo / G : -1;
    const int pos_hi = r_hi < rows ? pos_first + r_hi / G : -1;
    // the warp's own key range: nothing above its last row's position, nothing a window hides
    const int w_last_row = min(rows, warp * 16 + 16) - 1;
    const int w_pos_max = w_last_row >= warp * 16 ? pos_first + w_last_row / G : -1;
    const int w_pos_min = pos_first + (warp * 16) / G;

    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    float o[D / 8][4];
#pragma unroll
    for (int n = 0; n < D / 8; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) o[n][e] = 0.f;
    const float scale_log2 = scale * LOG2E;

    const int n_tiles = (pos_last - j_begin) / 64 + 1;
    PagedLoader<D, 64, 128> loader;
    loader.init(tid, kvh, Hkv, P, p_shift);
    auto issue = [&](int it) {
        const uint32_t base = smem + (uint32_t)(it & 1) * 2 * TILE_BYTES;
        const int j0 = j_begin + it * 64;
        if (p_shift >= 0) {
            // (pages looked up one tile ahead, as in the decode kernel)
            loader.issue_looked_up(base, base + TILE_BYTES, pool, j0, lo, pos_last);
            if (it + 1 < n_tiles) loader.lookup(bt_row, j0 + 64, lo, pos_last);
        } else {
            load_tile<D>(base, pool, bt_row, j0, 64, lo, pos_last, kvh, Hkv, P, 0, tid, 128);
            load_tile<D>(base + TILE_BYTES, pool, bt_row, j0, 64, lo, pos_last, kvh, Hkv, P, 1, tid, 128);
        }
        cp_async_commit();
    };
    if (p_shift >= 0) loader.lookup(bt_row, j_begin, lo, pos_last);
    issue(0);
    for (int it = 0; it < n_tiles; ++it) {
        cp_async_wait<0>();
        __syncthreads();
        if (it + 1 < n_tiles) issue(it + 1);
        const int j0 = j_begin + it * 64;
        const bool active = w_pos_max >= j0 && (window <= 0 || j0 + 63 > w_pos_min - window);
        if (active) {
            const bool need_mask = (j0 + 63 > w_pos_min) || (window > 0 && j0 <= w_pos_max - window) ||
                                   pos_lo < 0 || pos_hi < 0;
            const uint32_t base = smem + (uint32_t)(it & 1) * 2 * TILE_BYTES;
            warp_block<D, 64>(qf, base, base + TILE_BYTES, j0, pos_lo, pos_hi, window, scale_log2,
                              need_mask, m, l, o);
        }
    }
    // finish: row sums over the 4 threads of a row, normalise, store
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        l[h] += __shfl_xor_sync(0xffffffffu, l[h], 1);
        l[h] += __shfl_xor_sync(0xffffffffu, l[h], 2);
    }
    const int t = lane & 3;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int r = warp * 16 + g + 8 * half;
        if (r >= rows) continue;
        const float inv = l[half] > 0.f ? 1.0f / l[half] : 0.f;
        __nv_bfloat16* dst = out + ((size_t)(tok0 + r / G) * H + kvh * G + r % G) * D;
        const float gs = head_gate_of(gate, ldg, tok0 + r / G, kvh * G + r % G);
#pragma unroll
        for (int n = 0; n < D / 8; ++n) {
            uint32_t v = pack_bf16(o[n][half * 2] * inv, o[n][half * 2 + 1] * inv);
            if (gate != nullptr) {
                const float2 f = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&v));
                v = pack_bf16(f.x * gs, f.y * gs);
            }
            *reinterpret_cast<uint32_t*>(dst + n * 8 + 2 * t) = v;
        }
    }
}

// ---------------------------------------------------------------------------------------------
// decode: one token per sequence; CTA (token, kv head, split); warps take alternate 32-key tiles
// ---------------------------------------------------------------------------------------------
template <int D>
__global__ void __launch_bounds__(128)
attn_decode_mma_kernel(const __nv_bfloat16* q, const __nv_bfloat16* pool,
                       __nv_bfloat16* out, const int* positions,
                       const int* tok_seq, const int* block_table,
                       int bt_stride, const int* tok_index, int H, int Hkv, int P,
                       int window, float scale, int nsplit, float* part_o,
                       float* part_ml, int p_shift, const __nv_bfloat16* gate, int64_t ldg) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ __align__(128) unsigned char smem_raw[];
    constexpr int TILE_BYTES = 32 * D * 2;           // one warp's 32 keys
    const int G = H / Hkv;
    const int i = blockIdx.x;                        // which decode token
    const int kvh = blockIdx.y, split = blockIdx.z;
    const int tok = tok_index != nullptr ? tok_index[i] : i;     // null: token i is sequence i's one token
    if (tok < 0) return;         // an unused entry of a fixed-length list (captured steps)
    const int seq = tok_seq[tok];
    const int pos = positions[tok];
    const int* bt_row = block_table + (size_t)seq * bt_stride;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const int j_begin = (lo / 32) * 32;
    const int tiles = (pos - j_begin) / 32 + 1;
    const int per_split = (tiles + nsplit - 1) / nsplit;
    const int t_begin = split * per_split, t_end = min(tiles, t_begin + per_split);

    uint32_t qf[D / 16][4];
    load_q<D>(qf, q, 0, G, tok, G, H, kvh * G);      // rows 0..G-1 are the group's heads
    const int pos_lo = g < G ? pos : -1, pos_hi = g + 8 < G ? pos : -1;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    float o[D / 8][4];
#pragma unroll
    for (int n = 0; n < D / 8; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) o[n][e] = 0.f;
    const float scale_log2 = scale * LOG2E;

    // the warp's private double buffer: [stage][K|V][32][D]
    const uint32_t wbase = smem_u32(smem_raw) + (uint32_t)warp * 4 * TILE_BYTES;
    PagedLoader<D, 32, 32> loader;
    loader.init(lane, kvh, Hkv, P, p_shift);
    auto issue = [&](int tile, int stage) {
        const uint32_t base = wbase + (uint32_t)stage * 2 * TILE_BYTES;
        const int j0 = j_begin + tile * 32;
        if (p_shift >= 0) {
            // the pages of this tile were looked up when the tile before it was issued; now the
            // next tile's are, so that no copy waits for a block-table entry
            loader.issue_looked_up(base, base + TILE_BYTES, pool, j0, lo, pos);
            if (tile + 4 < t_end) loader.lookup(bt_row, j0 + 4 * 32, lo, pos);
        } else {
            load_tile<D>(base, pool, bt_row, j0, 32, lo, pos, kvh, Hkv, P, 0, lane, 32);
            load_tile<D>(base + TILE_BYTES, pool, bt_row, j0, 32, lo, pos, kvh, Hkv, P, 1, lane, 32);
        }
        cp_async_commit();
    };
    int stage = 0;
    if (t_begin + warp < t_end) {
        if (p_shift >= 0) loader.lookup(bt_row, j_begin + (t_begin + warp) * 32, lo, pos);
        issue(t_begin + warp, 0);
    }
    for (int tile = t_begin + warp; tile < t_end; tile += 4) {
        const bool more = tile + 4 < t_end;
        if (more) issue(tile + 4, stage ^ 1);
        if (more) cp_async_wait<1>(); else cp_async_wait<0>();
        __syncwarp();
        const int j0 = j_begin + tile * 32;
        const bool need_mask = true;                 // rows past G are always masked
        const uint32_t base = wbase + (uint32_t)stage * 2 * TILE_BYTES;
        warp_block<D, 32>(qf, base, base + TILE_BYTES, j0, pos_lo, pos_hi, window, scale_log2,
                          need_mask, m, l, o);
        __syncwarp();
        stage ^= 1;
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        l[h] += __shfl_xor_sync(0xffffffffu, l[h], 1);
        l[h] += __shfl_xor_sync(0xffffffffu, l[h], 2);
    }
    // merge the four warps through shared memory (the K/V buffers are done with)
    __syncthreads();
    float* sm_o = reinterpret_cast<float*>(smem_raw);              // [4][16][D]
    float* sm_ml = sm_o + 4 * 16 * D;                              // [4][16][2]
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int r = g + 8 * half;
#pragma unroll
        for (int n = 0; n < D / 8; ++n) {
            sm_o[(warp * 16 + r) * D + n * 8 + 2 * t] = o[n][half * 2];
            sm_o[(warp * 16 + r) * D + n * 8 + 2 * t + 1] = o[n][half * 2 + 1];
        }
        if (t == 0) {
            sm_ml[(warp * 16 + r) * 2] = m[half];
            sm_ml[(warp * 16 + r) * 2 + 1] = l[half];
        }
    }
    __syncthreads();
    for (int idx = tid; idx < G * D; idx += 128) {
        const int r = idx / D, c = idx % D;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) M = fmaxf(M, sm_ml[(w * 16 + r) * 2]);
        float L = 0.f, acc = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float mw = sm_ml[(w * 16 + r) * 2];
            const float f = mw == -INFINITY ? 0.f : fast_exp2((mw - M) * scale_log2);
            L += sm_ml[(w * 16 + r) * 2 + 1] * f;
            acc += sm_o[(w * 16 + r) * D + c] * f;
        }
        const int head = kvh * G + r;
        if (nsplit == 1) {
            float y = round_as<__nv_bfloat16>(L > 0.f ? acc / L : 0.f);
            if (gate != nullptr) y *= head_gate_of(gate, ldg, tok, head);
            out[((size_t)tok * H + head) * D + c] = __float2bfloat16_rn(y);
        } else {
            const size_t slot = ((size_t)i * H + head) * nsplit + split;
            part_o[slot * D + c] = acc;
            if (c == 0) {
                part_ml[slot * 2] = M;
                part_ml[slot * 2 + 1] = L;
            }
        }
    }
}

template <int D>
__global__ void attn_decode_merge_kernel(const float* part_o,
                                         const float* part_ml,
                                         __nv_bfloat16* out,
                                         const int* tok_index, int H, int nsplit,
                                         float scale, const __nv_bfloat16* gate, int64_t ldg) {
    pdl_launch_dependents();
    pdl_wait();
    const int i = blockIdx.x, head = blockIdx.y, c = threadIdx.x;
    const int tok = tok_index != nullptr ? tok_index[i] : i;
    if (tok < 0) return;                 // an unused entry of a fixed-length list (captured steps)
    const size_t base = ((size_t)i * H + head) * nsplit;
    const float scale_log2 = scale * LOG2E;
    float M = -INFINITY;
    for (int s = 0; s < nsplit; ++s) M = fmaxf(M, part_ml[(base + s) * 2]);
    float L = 0.f, acc = 0.f;
    for (int s = 0; s < nsplit; ++s) {
        const float ms = part_ml[(base + s) * 2];
        const float f = ms == -INFINITY ? 0.f : fast_exp2((ms - M) * scale_log2);
        L += part_ml[(base + s) * 2 + 1] * f;
        acc += part_o[(base + s) * D + c] * f;
    }
    float y = round_as<__nv_bfloat16>(L > 0.f ? acc / L : 0.f);
    if (gate != nullptr) y *= head_gate_of(gate, ldg, tok, head);
    out[((size_t)tok * H + head) * D + c] = __float2bfloat16_rn(y);
}

// ---------------------------------------------------------------------------------------------
// decode, a layer's whole attention core in one kernel: the q/k norm, the rotation and the cache
// write of the new key and value (qk_rope.cu's formulas, to the bit), the split attention above,
// the merge of the splits by whichever CTA of a (token, KV head) finishes last, and the per-head
// output gate  out = round(round(o) * round(sigmoid(g))).
//   - Everything a CTA can know before the kernel in front of it has finished is asked for ahead
//     of the dependency wait: the page numbers, the first key/value tiles (earlier steps wrote
//     them; the tile that holds this step's position is never among them) and the angles.
//   - The new key and value never make the trip through memory: the CTA whose range holds the
//     position writes them to the cache for later steps, and every CTA that needs them patches
//     them into its shared-memory tile.
//   - `tickets` [n * Hkv] are zero between launches: each CTA adds one after its partial result is
//     visible, the one that draws the last number merges and puts the zero back.
// ---------------------------------------------------------------------------------------------
struct DecodeFused {
    const __nv_bfloat16* qkv;       // [n, >= (H + 2 Hkv) D] raw projection rows (q heads only if !write_kv)
    int64_t ldq;
    __nv_bfloat16* pool;
    __nv_bfloat16* out;             // [n, H, D]
    const float* wq;                // null: no q/k norm
    const float* wk;
    float eps;
    const float* inv_freq;          // [R / 2]
    int R;
    const __nv_bfloat16* gate;      // [n, >= H] rows ldg apart; null: no gate
    int64_t ldg;
    const int* positions;
    const int* tok_seq;
    const int* block_table;
    int bt_stride;
    int H, Hkv, P, window;
    float scale;
    int nsplit;
    float* part_o;
    float* part_ml;
    int* tickets;
    int p_shift;
    int write_kv;                   // 0: the layer reads another layer's cache, which holds this step's key already
};

template <int D>
__global__ void __launch_bounds__(128) attn_decode_fused_kernel(const DecodeFused a) {
    pdl_launch_dependents();
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __shared__ int s_last;
    constexpr int TILE_BYTES = 32 * D * 2;                   // one warp's 32 keys
    constexpr int STAGING = 4 * 2 * 2 * TILE_BYTES;          // [warp][stage][K|V]; later the warps' merge
    constexpr int QS = D + 8;                                // row stride of the query tile (no bank conflicts)
    __nv_bfloat16* sm_q = reinterpret_cast<__nv_bfloat16*>(smem_raw + STAGING);     // [G][QS]
    __nv_bfloat16* sm_new = sm_q + 16 * QS;                                        // the new key, the new value
    float* sm_cs = reinterpret_cast<float*>(sm_new + 2 * D);                       // [D/2] cos, [D/2] sin
    float* sm_sn = sm_cs + D / 2;
    const int H = a.H, Hkv = a.Hkv, P = a.P, window = a.window, nsplit = a.nsplit;
    const int G = H / Hkv;
    const int i = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
    const int tok = i;
    const int seq = a.tok_seq[tok];
    const int pos = a.positions[tok];
    const int* bt_row = a.block_table + (size_t)seq * a.bt_stride;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const int j_begin = (lo / 32) * 32;
    const int tiles = (pos - j_begin) / 32 + 1;
    const int per_split = (tiles + nsplit - 1) / nsplit;
    const int t_begin = split * per_split, t_end = min(tiles, t_begin + per_split);
    const int last_tile = tiles - 1;                         // the tile that holds position `pos`
    const int j_last = a.write_kv ? pos - 1 : pos;           // the last key that comes from the cache
    const bool owner = a.write_kv && t_begin <= last_tile && last_tile < t_end;
    size_t cache_row = 0;
    if (owner) {
        const int page = TK_PAGE(TK_K_QK_ROPE, bt_row[a.p_shift >= 0 ? pos >> a.p_shift : pos / P]);
        cache_row = (size_t)page * 2 * Hkv * P + (a.p_shift >= 0 ? pos & (P - 1) : pos % P);
    }
    const int half = a.R >> 1;
    for (int k = tid; k < half; k += 128) {
        float s_, c_;
        sincosf((float)pos * a.inv_freq[k], &s_, &c_);
        sm_cs[k] = round_as<__nv_bfloat16>(c_);
        sm_sn[k] = round_as<__nv_bfloat16>(s_);
    }

    // the warp's private double buffer: [stage][K|V][32][D]
    const uint32_t wbase = smem_u32(smem_raw) + (uint32_t)warp * 4 * TILE_BYTES;
    PagedLoader<D, 32, 32> loader;
    loader.init(lane, kvh, Hkv, P, a.p_shift);
    auto issue = [&](int tile, int stage) {
        const uint32_t base = wbase + (uint32_t)stage * 2 * TILE_BYTES;
        const int j0 = j_begin + tile * 32;
        if (a.p_shift >= 0) {
            loader.issue_looked_up(base, base + TILE_BYTES, a.pool, j0, lo, j_last);
            if (tile + 4 < t_end) loader.lookup(bt_row, j0 + 4 * 32, lo, pos);
        } else {
            load_tile<D>(base, a.pool, bt_row, j0, 32, lo, j_last, kvh, Hkv, P, 0, lane, 32);
            load_tile<D>(base + TILE_BYTES, a.pool, bt_row, j0, 32, lo, j_last, kvh, Hkv, P, 1, lane, 32);
        }
        cp_async_commit();
    };
    const int first = t_begin + warp;
    const bool deferred = first == last_tile;                // this step writes into that tile
    if (first < t_end && !deferred) {
        if (a.p_shift >= 0) loader.lookup(bt_row, j_begin + first * 32, lo, pos);
        issue(first, 0);
    }
    pdl_wait();
    __syncthreads();                                         // the angles are in place

    // the group's query heads, then the new key, then the new value: a head over LPH lanes
    {
        constexpr int LPH = D / 8, HPP = 32 / LPH;
        const int sub = lane / LPH, c = (lane % LPH) * 8;
        const int jobs = G + (a.write_kv ? 2 : 0);
        const int half_lanes = half / 8;
        const int partner = c < half ? lane + half_lanes : (c < a.R ? lane - half_lanes : lane);
        const __nv_bfloat16* row = a.qkv + (size_t)tok * a.ldq;
        for (int j0 = warp * HPP; j0 < jobs; j0 += 4 * HPP) {
            const int job = j0 + sub;
            const bool live = job < jobs;
            const __nv_bfloat16* src = row;
            const float* w = nullptr;
            bool rotate = true;
            if (job < G) {
                src = row + (size_t)(kvh * G + job) * D;
                w = a.wq;
            } else if (job == G) {
                src = row + (size_t)(H + kvh) * D;
                w = a.wk;
            } else {
                src = row + (size_t)(H + Hkv + kvh) * D;
                rotate = false;
            }
            uint4 raw = make_uint4(0u, 0u, 0u, 0u);
            if (live) raw = *reinterpret_cast<const uint4*>(src + c);
            const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(&raw);
            float v[8];
            float ss = 0.f;
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                v[k] = __bfloat162float(e[k]);
                ss += v[k] * v[k];
            }
            for (int o = LPH >> 1; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            if (rotate && w != nullptr) {
                const float rstd = 1.0f / sqrtf(ss / (float)D + a.eps);
#pragma unroll
                for (int k = 0; k < 8; ++k)
                    v[k] = round_as<__nv_bfloat16>(round_as<__nv_bfloat16>(v[k] * rstd) * w[c + k]);
            }
            float pv[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) pv[k] = __shfl_sync(0xffffffffu, v[k], partner);
            if (!live) continue;
            uint4 packed = raw;
            if (rotate) {
                __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(&packed);
                const int i0 = c < half ? c : c - half;
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    float r = v[k];
                    if (c < a.R) r = r * sm_cs[i0 + k] + (c < half ? -pv[k] : pv[k]) * sm_sn[i0 + k];
                    o[k] = __float2bfloat16_rn(r);
                }
            }
            if (job < G) {
                *reinterpret_cast<uint4*>(sm_q + job * QS + c) = packed;
            } else {
                *reinterpret_cast<uint4*>(sm_new + (job - G) * D + c) = packed;
                if (owner)
                    *reinterpret_cast<uint4*>(a.pool + (cache_row + (size_t)((job - G) * Hkv + kvh) * P) * D + c) = packed;
            }
        }
    }
    __syncthreads();

    uint32_t qf[D / 16][4];                                  // rows 0..G-1 are the group's heads
#pragma unroll
    for (int hf = 0; hf < 2; ++hf) {
        const int r = g + 8 * hf;
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
            uint32_t ql = 0u, qh = 0u;
            if (r < G) {
                ql = *reinterpret_cast<const uint32_t*>(sm_q + r * QS + ks * 16 + 2 * t);
                qh = *reinterpret_cast<const uint32_t*>(sm_q + r * QS + ks * 16 + 8 + 2 * t);
            }
            qf[ks][hf] = ql;
            qf[ks][hf + 2] = qh;
        }
    }
    const int pos_lo = g < G ? pos : -1, pos_hi = g + 8 < G ? pos : -1;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    float o[D / 8][4];
#pragma unroll
    for (int n = 0; n < D / 8; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) o[n][e] = 0.f;
    const float scale_log2 = a.scale * LOG2E;

    if (first < t_end && deferred) {
        if (a.p_shift >= 0) loader.lookup(bt_row, j_begin + first * 32, lo, pos);
        issue(first, 0);
    }
    int stage = 0;
    for (int tile = first; tile < t_end; tile += 4) {
        const bool more = tile + 4 < t_end;
        if (more) issue(tile + 4, stage ^ 1);
        if (more) cp_async_wait<1>(); else cp_async_wait<0>();
        __syncwarp();
        const int j0 = j_begin + tile * 32;
        const uint32_t off = (uint32_t)warp * 4 * TILE_BYTES + (uint32_t)stage * 2 * TILE_BYTES;
        if (a.write_kv && tile == last_tile) {
            // this step's key and value: into their row of the tile (the copies left it zero)
            constexpr int LPH = D / 8;
            if (lane < 2 * LPH) {
                const int which = lane / LPH, ch = lane % LPH;
                const uint4 nv = *reinterpret_cast<const uint4*>(sm_new + which * D + ch * 8);
                *reinterpret_cast<uint4*>(smem_raw + off + which * TILE_BYTES + tile_off<D>(pos - j0, ch)) = nv;
            }
            __syncwarp();
        }
        const uint32_t base = smem_u32(smem_raw) + off;
        warp_block<D, 32>(qf, base, base + TILE_BYTES, j0, pos_lo, pos_hi, window, scale_log2, true, m, l, o);
        __syncwarp();
        stage ^= 1;
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        l[h] += __shfl_xor_sync(0xffffffffu, l[h], 1);
        l[h] += __shfl_xor_sync(0xffffffffu, l[h], 2);
    }
    // merge the four warps through shared memory (the K/V buffers are done with)
    __syncthreads();
    float* sm_o = reinterpret_cast<float*>(smem_raw);              // [4][16][D]
    float* sm_ml = sm_o + 4 * 16 * D;                              // [4][16][2]
#pragma unroll
    for (int hf = 0; hf < 2; ++hf) {
        const int r = g + 8 * hf;
#pragma unroll
        for (int n = 0; n < D / 8; ++n) {
            sm_o[(warp * 16 + r) * D + n * 8 + 2 * t] = o[n][hf * 2];
            sm_o[(warp * 16 + r) * D + n * 8 + 2 * t + 1] = o[n][hf * 2 + 1];
        }
        if (t == 0) {
            sm_ml[(warp * 16 + r) * 2] = m[hf];
            sm_ml[(warp * 16 + r) * 2 + 1] = l[hf];
        }
    }
    __syncthreads();
    // one finished element: rounded as the attention's output, gated, rounded again
    auto finish = [&](int head, int c, float val) {
        float y = round_as<__nv_bfloat16>(val);
        if (a.gate != nullptr) {
            const float gv = __bfloat162float(a.gate[(size_t)tok * a.ldg + head]);
            y *= round_as<__nv_bfloat16>(1.0f / (1.0f + expf(-gv)));
        }
        a.out[((size_t)tok * H + head) * D + c] = __float2bfloat16_rn(y);
    };
    for (int idx = tid; idx < G * D; idx += 128) {
        const int r = idx / D, c = idx % D;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) M = fmaxf(M, sm_ml[(w * 16 + r) * 2]);
        float L = 0.f, acc = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float mw = sm_ml[(w * 16 + r) * 2];
            const float f = mw == -INFINITY ? 0.f : fast_exp2((mw - M) * scale_log2);
            L += sm_ml[(w * 16 + r) * 2 + 1] * f;
            acc += sm_o[(w * 16 + r) * D + c] * f;
        }
        const int head = kvh * G + r;
        if (nsplit == 1) {
            finish(head, c, L > 0.f ? acc / L : 0.f);
        } else {
            const size_t slot = ((size_t)i * H + head) * nsplit + split;
            a.part_o[slot * D + c] = acc;
            if (c == 0) {
                a.part_ml[slot * 2] = M;
                a.part_ml[slot * 2 + 1] = L;
            }
        }
    }
    if (nsplit == 1) return;
    // the last CTA of this (token, KV head) to get here merges the splits
    __threadfence();
    __syncthreads();
    if (tid == 0) s_last = atomicAdd(&a.tickets[i * Hkv + kvh], 1) == nsplit - 1;
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    // every split's (maximum, sum) of the group's heads in one trip, then each head's weights
    float* sm_f = reinterpret_cast<float*>(smem_raw);            // [G][nsplit] maxima, then weights
    float* sm_l = sm_f + G * nsplit;                             // [G][nsplit] sums
    float* sm_inv = sm_l + G * nsplit;                           // [G] 1 / total, 0 for an empty row
    for (int idx = tid; idx < G * nsplit; idx += 128) {
        const int r = idx / nsplit, s = idx % nsplit;
        const float2 ml = __ldcg(reinterpret_cast<const float2*>(a.part_ml) + ((size_t)i * H + kvh * G + r) * nsplit + s);
        sm_f[idx] = ml.x;
        sm_l[idx] = ml.y;
    }
    __syncthreads();
    for (int r = warp; r < G; r += 4) {
        float M = -INFINITY;
        for (int s = lane; s < nsplit; s += 32) M = fmaxf(M, sm_f[r * nsplit + s]);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
        for (int s = lane; s < nsplit; s += 32) {
            const float ms = sm_f[r * nsplit + s];
            sm_f[r * nsplit + s] = ms == -INFINITY ? 0.f : fast_exp2((ms - M) * scale_log2);
        }
        // the sum runs over the splits in order, as the element loop below and the merge kernel do
        __syncwarp();
        if (lane == 0) {
            float tot = 0.f;
            for (int s = 0; s < nsplit; ++s) tot += sm_l[r * nsplit + s] * sm_f[r * nsplit + s];
            sm_inv[r] = tot;
        }
    }
    __syncthreads();
    constexpr int PER = 16 * D / 128;                            // elements a thread may own (G <= 16)
    float acc[PER];
#pragma unroll
    for (int k = 0; k < PER; ++k) acc[k] = 0.f;
    for (int s0 = 0; s0 < nsplit; s0 += 4) {
        float got[PER][4];
#pragma unroll
        for (int k = 0; k < PER; ++k) {
            const int idx = tid + k * 128;
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                got[k][u] = 0.f;
                if (idx < G * D && s0 + u < nsplit)
                    got[k][u] = __ldcg(&a.part_o[(((size_t)i * H + kvh * G + idx / D) * nsplit + s0 + u) * D + idx % D]);
            }
        }
#pragma unroll
        for (int k = 0; k < PER; ++k) {
            const int idx = tid + k * 128;
            if (idx >= G * D) continue;
#pragma unroll
            for (int u = 0; u < 4; ++u)
                if (s0 + u < nsplit) acc[k] += got[k][u] * sm_f[(idx / D) * nsplit + s0 + u];
        }
    }
#pragma unroll
    for (int k = 0; k < PER; ++k) {
        const int idx = tid + k * 128;
        if (idx >= G * D) continue;
        const int r = idx / D;
        const float L = sm_inv[r];
        finish(kvh * G + r, idx % D, L > 0.f ? acc[k] / L : 0.f);
    }
    if (tid == 0) a.tickets[i * Hkv + kvh] = 0;
}

// log2 of a power-of-two page size, else -1 (the kernels then divide per 16-byte request)
int page_shift(int P) {
    if (P <= 0 || (P & (P - 1))) return -1;
    int s = 0;
    while ((1 << s) < P) ++s;
    return s;
}

bool mma_shape_ok(int H, int Hkv, int D) {
    if (Hkv <= 0 || H % Hkv) return false;
    const int G = H / Hkv;
    return (D == 64 || D == 128) && G >= 1 && G <= 16 && (G & (G - 1)) == 0;
}

}  // namespace

// 1 when the tensor-core kernels take this shape (bfloat16, head size 64 or 128, a group of
// 1, 2, 4, 8 or 16 query heads per KV head); otherwise the generic kernel is the one to call.
TK_API int tk_attn_mma_supported(int H, int Hkv, int D) { return mma_shape_ok(H, Hkv, D) ? 1 : 0; }

// Tokens per tile the prefill kernel expects: 64 rows / G heads.
TK_API int tk_attn_prefill_mma_tokens(int H, int Hkv) { return 64 / (H / Hkv); }

TK_API int tk_attn_prefill_mma(const void* q, const void* kv_pool, void* out, const int* positions,
                               const int* tok_seq, const int* block_table, int bt_stride,
                               const int* tile_tok0, const int* tile_ntok, int n_tiles, int H,
                               int Hkv, int D, int P, int window, float scale, const void* gate,
                               int64_t ldg, cudaStream_t stream) {
    TK_CHECK_ARG(mma_shape_ok(H, Hkv, D), "attn_prefill_mma: shape H=%d Hkv=%d D=%d is not taken "
                 "(head size 64 or 128, group a power of two up to 16)", H, Hkv, D);
    TK_CHECK_ARG(P > 0 && n_tiles >= 0, "attn_prefill_mma: bad page size or tile count");
    if (n_tiles == 0) return 0;
    dim3 grid(n_tiles * Hkv);
    const size_t smem = 2 * 2 * 64 * (size_t)D * 2;
    auto q_ = (const __nv_bfloat16*)q;
    auto p_ = (const __nv_bfloat16*)kv_pool;
    auto o_ = (__nv_bfloat16*)out;
    auto g_ = (const __nv_bfloat16*)gate;
    if (D == 64) {
        cudaFuncSetAttribute(attn_prefill_mma_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        tk_launch(attn_prefill_mma_kernel<64>, dim3(grid), dim3(128), smem, stream, q_, p_, o_, positions, tok_seq, block_table,
                                                                 bt_stride, tile_tok0, tile_ntok, H, Hkv, P, window, scale, page_shift(P), g_, ldg);
    } else {
        cudaFuncSetAttribute(attn_prefill_mma_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        tk_launch(attn_prefill_mma_kernel<128>, dim3(grid), dim3(128), smem, stream, q_, p_, o_, positions, tok_seq, block_table,
                                                                  bt_stride, tile_tok0, tile_ntok, H, Hkv, P, window, scale, page_shift(P), g_, ldg);
    }
    TK_CHECK_LAUNCH("attn_prefill_mma");
    return 0;
}

// Floats of scratch the decode kernel needs for `n` tokens split `nsplit` ways:
// part_o [n, H, nsplit, D] then part_ml [n, H, nsplit, 2] (nothing when nsplit is 1).
TK_API int64_t tk_attn_decode_mma_scratch(int n, int H, int D, int nsplit) {
    return nsplit <= 1 ? 0 : (int64_t)n * H * nsplit * (D + 2);
}

TK_API int tk_attn_decode_mma(const void* q, const void* kv_pool, void* out, const int* positions,
                              const int* tok_seq, const int* block_table, int bt_stride,
                              const int* tok_index, int n, int H, int Hkv, int D, int P, int window,
                              float scale, int nsplit, float* scratch, const void* gate, int64_t ldg,
                              cudaStream_t stream) {
    TK_CHECK_ARG(mma_shape_ok(H, Hkv, D), "attn_decode_mma: shape H=%d Hkv=%d D=%d is not taken "
                 "(head size 64 or 128, group a power of two up to 16)", H, Hkv, D);
    TK_CHECK_ARG(P > 0 && n >= 0 && nsplit >= 1 && nsplit <= 65535, "attn_decode_mma: bad sizes");
    if (n == 0) return 0;
    TK_CHECK_ARG(nsplit == 1 || scratch != nullptr, "attn_decode_mma: %d splits need scratch memory", nsplit);
    float* part_o = scratch;
    float* part_ml = scratch ? scratch + (size_t)n * H * nsplit * D : nullptr;
    dim3 grid(n, Hkv, nsplit);
    // K/V staging: 4 warps x 2 stages x (K, V) x 32 keys; the merge reuses it as [4][16][D+2] floats
    const size_t staging = 4 * 2 * 2 * 32 * (size_t)D * 2;
    const size_t merge = 4 * 16 * ((size_t)D + 2) * sizeof(float);
    const size_t smem = staging > merge ? staging : merge;
    auto q_ = (const __nv_bfloat16*)q;
    auto p_ = (const __nv_bfloat16*)kv_pool;
    auto o_ = (__nv_bfloat16*)out;
    auto g_ = (const __nv_bfloat16*)gate;
    if (D == 64) {
        cudaFuncSetAttribute(attn_decode_mma_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        tk_launch(attn_decode_mma_kernel<64>, dim3(grid), dim3(128), smem, stream, q_, p_, o_, positions, tok_seq, block_table, bt_stride,
                                                                tok_index, H, Hkv, P, window, scale, nsplit, part_o, part_ml, page_shift(P), g_, ldg);
        TK_CHECK_LAUNCH("attn_decode_mma");
        if (nsplit > 1)
            tk_launch(attn_decode_merge_kernel<64>, dim3(dim3(n, H)), dim3(64), 0, stream, part_o, part_ml, o_, tok_index, H, nsplit, scale, g_, ldg);
    } else {
        cudaFuncSetAttribute(attn_decode_mma_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        tk_launch(attn_decode_mma_kernel<128>, dim3(grid), dim3(128), smem, stream, q_, p_, o_, positions, tok_seq, block_table, bt_stride,
                                                                 tok_index, H, Hkv, P, window, scale, nsplit, part_o, part_ml, page_shift(P), g_, ldg);
        TK_CHECK_LAUNCH("attn_decode_mma");
        if (nsplit > 1)
            tk_launch(attn_decode_merge_kernel<128>, dim3(dim3(n, H)), dim3(128), 0, stream, part_o, part_ml, o_, tok_index, H, nsplit, scale, g_, ldg);
    }
    TK_CHECK_LAUNCH("attn_decode_merge");
    return 0;
}

// 1 when tk_attn_decode_fused takes this shape: what the tensor-core kernels take, and a rotation
// whose halves are whole 16-byte chunks.
TK_API int tk_attn_decode_fused_supported(int H, int Hkv, int D, int R) {
    return mma_shape_ok(H, Hkv, D) && R >= 0 && R <= D && R % 16 == 0 ? 1 : 0;
}

// The most splits tk_attn_decode_fused takes: the merging CTA holds every split's maximum and sum
// of the group's heads in the shared memory its key/value tiles left.
TK_API int tk_attn_decode_fused_max_splits(int H, int Hkv, int D) {
    if (!mma_shape_ok(H, Hkv, D)) return 0;
    const int G = H / Hkv;
    const int floats = 4 * 2 * 2 * 32 * D * 2 / 4;
    const int most = (floats - G) / (2 * G);
    return most < 65535 ? most : 65535;
}

// A decode step's attention for `n` sequences of one token each, from the raw projection rows
// `qkv` [n, (H + 2 Hkv) D] (rows `ldq` elements apart) to the gated heads' outputs `out`
// [n, H, D]: q/k norm (wq, wk null: none), rotate-half rotation of the first R columns by
// position x inv_freq, the new key and value into the cache (write_kv 0: the layer has none of
// its own and `qkv` holds queries only), attention split `nsplit` ways, merge, gate (null: none).
// `scratch`: tk_attn_decode_mma_scratch floats (nsplit > 1); `tickets`: n * Hkv ints that are zero
// and are zero again when the kernel has finished. `carveout`: the share of the SM's memory (in
// percent of the most it can give) this launch would like as shared memory, -1 for the driver's
// choice. It matters to the kernels around this one more than to this one: an SM changes its
// split between shared memory and L1 only when it is empty, so a kernel that asks for another
// split than its neighbours cannot start under them, and the split it leaves behind is the L1 the
// next kernels' loads find.
TK_API int tk_attn_decode_fused(const void* qkv, int64_t ldq, void* kv_pool, void* out, const float* wq,
                                const float* wk, float eps, const float* inv_freq, int R,
                                const void* gate, int64_t ldg, const int* positions, const int* tok_seq,
                                const int* block_table, int bt_stride, int n, int H, int Hkv, int D, int P,
                                int window, float scale, int nsplit, float* scratch, int* tickets,
                                int write_kv, int carveout, cudaStream_t stream) {
    TK_CHECK_ARG(tk_attn_decode_fused_supported(H, Hkv, D, R),
                 "attn_decode_fused: shape H=%d Hkv=%d D=%d rotary %d is not taken (head size 64 or 128, "
                 "group a power of two up to 16, rotary width a multiple of 16)", H, Hkv, D, R);
    TK_CHECK_ARG(P > 0 && n >= 0 && nsplit >= 1, "attn_decode_fused: bad sizes");
    TK_CHECK_ARG(nsplit <= tk_attn_decode_fused_max_splits(H, Hkv, D), "attn_decode_fused: %d splits, at most %d",
                 nsplit, tk_attn_decode_fused_max_splits(H, Hkv, D));
    TK_CHECK_ARG(ldq % 8 == 0 && (uintptr_t)qkv % 16 == 0 && (uintptr_t)kv_pool % 16 == 0,
                 "attn_decode_fused: projection rows and the cache must be 16-byte aligned");
    TK_CHECK_ARG((wq == nullptr) == (wk == nullptr) || !write_kv, "attn_decode_fused: q and k norms come together");
    TK_CHECK_ARG(inv_freq != nullptr || R == 0, "attn_decode_fused: a rotation needs its frequencies");
    if (n == 0) return 0;
    TK_CHECK_ARG(nsplit == 1 || (scratch != nullptr && tickets != nullptr),
                 "attn_decode_fused: %d splits need scratch memory and tickets", nsplit);
    DecodeFused a;
    a.qkv = (const __nv_bfloat16*)qkv;
    a.ldq = ldq;
    a.pool = (__nv_bfloat16*)kv_pool;
    a.out = (__nv_bfloat16*)out;
    a.wq = wq;
    a.wk = wk;
    a.eps = eps;
    a.inv_freq = inv_freq;
    a.R = R;
    a.gate = (const __nv_bfloat16*)gate;
    a.ldg = ldg;
    a.positions = positions;
    a.tok_seq = tok_seq;
    a.block_table = block_table;
    a.bt_stride = bt_stride;
    a.H = H;
    a.Hkv = Hkv;
    a.P = P;
    a.window = window;
    a.scale = scale;
    a.nsplit = nsplit;
    a.part_o = scratch;
    a.part_ml = scratch ? scratch + (size_t)n * H * nsplit * D : nullptr;
    a.tickets = tickets;
    a.p_shift = page_shift(P);
    a.write_kv = write_kv ? 1 : 0;
    dim3 grid(n, Hkv, nsplit);
    // K/V staging (the warps' merge reuses it), the query tile, the new key and value, cos and sin
    const size_t smem = 4 * 2 * 2 * 32 * (size_t)D * 2 + 16 * ((size_t)D + 8) * 2 + 2 * (size_t)D * 2 +
                        (size_t)D * sizeof(float);
    const int prefer = carveout >= 0 && carveout <= 100 ? carveout : (int)cudaSharedmemCarveoutDefault;
    if (D == 64) {
        cudaFuncSetAttribute(attn_decode_fused_kernel<64>, cudaFuncAttributePreferredSharedMemoryCarveout, prefer);
        cudaFuncSetAttribute(attn_decode_fused_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        tk_launch(attn_decode_fused_kernel<64>, dim3(grid), dim3(128), smem, stream, a);
    } else {
        cudaFuncSetAttribute(attn_decode_fused_kernel<128>, cudaFuncAttributePreferredSharedMemoryCarveout, prefer);
        cudaFuncSetAttribute(attn_decode_fused_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        tk_launch(attn_decode_fused_kernel<128>, dim3(grid), dim3(128), smem, stream, a);
    }
    TK_CHECK_LAUNCH("attn_decode_fused");
    return 0;
}

// ---------------------------------------------------------------------------------------------
// Split decode attention for callers that must not allocate (declared in no_alloc.h).
//
// tk_attn_decode_mma wants its scratch (the per-split partial results) from the caller, who
// normally gets it from an allocator. Some callers cannot: code that runs inside a CUDA stream
// capture it does not own, a latency-critical serving loop that has promised its memory pool
// to someone else, a host language binding without an allocator of its own. For them the same
// kernel runs on a fixed scratch that lives in the library image: a file-scope __device__ array.
// The array's name is only a host-side handle; the device address comes from
// cudaGetSymbolAddress, asked for once per device at that device's first call.
// ---------------------------------------------------------------------------------------------
namespace {
constexpr long long NOALLOC_SCRATCH_FLOATS = 2ll << 20;           // 8 MiB per device
static __device__ __align__(256) float g_decode_scratch[NOALLOC_SCRATCH_FLOATS];
constexpr int NOALLOC_MAX_DEVICES = 64;
float* g_decode_scratch_ptr[NOALLOC_MAX_DEVICES] = {};
}  // namespace

TK_API long long tk_attn_decode_mma_static_capacity() { return NOALLOC_SCRATCH_FLOATS; }

TK_API int tk_attn_decode_mma_static(const void* q, const void* kv_pool, void* out,
                                     const int* positions, const int* tok_seq,
                                     const int* block_table, int bt_stride, const int* tok_index,
                                     int n, int H, int Hkv, int D, int P, int window, float scale,
                                     int nsplit, cudaStream_t stream) {
    TK_CHECK_ARG(n >= 0 && H > 0 && D > 0 && nsplit >= 1, "attn_decode_mma_static: bad sizes");
    const long long need = tk_attn_decode_mma_scratch(n, H, D, nsplit);
    TK_CHECK_ARG(need <= NOALLOC_SCRATCH_FLOATS,
                 "attn_decode_mma_static: %d tokens x %d heads x %d splits x (%d + 2) = %lld floats of "
                 "scratch, the built-in array holds %lld; use fewer splits or tk_attn_decode_mma with "
                 "your own scratch", n, H, nsplit, D, need, (long long)NOALLOC_SCRATCH_FLOATS);
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    TK_CHECK_ARG(e == cudaSuccess && dev >= 0 && dev < NOALLOC_MAX_DEVICES,
                 "attn_decode_mma_static: cudaGetDevice: %s (device %d)", cudaGetErrorString(e), dev);
    if (g_decode_scratch_ptr[dev] == nullptr) {
        // once per device, with that device current: the symbol's address on *this* device
        float* p = nullptr;
        e = cudaGetSymbolAddress((void**)&p, g_decode_scratch);
        TK_CHECK_ARG(e == cudaSuccess && p != nullptr, "attn_decode_mma_static: cudaGetSymbolAddress: %s",
                     cudaGetErrorString(e));
        g_decode_scratch_ptr[dev] = p;
    }
    return tk_attn_decode_mma(q, kv_pool, out, positions, tok_seq, block_table, bt_stride, tok_index, n, H,
                              Hkv, D, P, window, scale, nsplit, g_decode_scratch_ptr[dev], nullptr, 0, stream);
}
