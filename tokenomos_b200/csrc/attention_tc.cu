// Paged prefill attention on the fifth-generation tensor cores, for bfloat16 and head size 64:
// S = Q K^T and O += P V are tcgen05.mma instructions with their accumulators in tensor memory;
// the online softmax runs on 128 threads, one query row each.
//
// A CTA takes up to 128 rows: 128 / G tokens of one sequence with the G query heads that share one
// KV head (row = token * G + head), and walks the keys in tiles of 64, this step's own keys
// included. Three groups of warps, coupled by mbarriers only:
//
//   warps 0-3  stage the tiles: Q once, then per tile K and V from the paged cache with cp.async
//              into 128-byte-swizzled K-major tiles (three stages of K and turned V). K is used as
//              it lands ([key][d] is the B operand of S = Q K^T). V must be contracted over its
//              keys, so the same warps turn the [key][d] tile into [d][key] with ldmatrix.trans +
//              stmatrix (8 x 8 blocks).
//   warp 8     one lane issues the MMAs: S_j (128 x 64 x 64) into one of two S accumulators, so
//              that S_{j+1} is computed while the softmax of tile j runs, and O += P_j V_j into
//              a third accumulator that lives in tensor memory for the whole walk.
//   warps 4-7  thread r owns row r: reads S_j from tensor memory into registers, masks (causal,
//              window), keeps a reference maximum and the row sum in 32-bit, and writes P_j as
//              bfloat16 into one of two A operand tiles of the second product, so that writing
//              P_j never waits for P_{j-1} V_{j-1}. The reference maximum
//              follows the true one lazily (see the softmax section); only when it is raised is
//              the accumulated output read, scaled and written back (tcgen05.ld / tcgen05.st).
//
// Masking, scale, rounding of P to bfloat16 and the unrounded row sum are those of the other
// attention kernels (Tokenomos kernels/attention/paged.py:67-76,150,267;
// models/blocks/attention.py:31-40,173). Keys past the tile's last position are never read.
//
// Every mbarrier wait is bounded (about a second, or until another thread has recorded an
// error); the kernel then leaves its loops, frees its tensor memory and returns, and
// tk_attn_prefill_tc_status() reports where it gave up.
#include <math.h>

#include "paged_tiles.cuh"
#include "tcgen05.cuh"

namespace {

constexpr int AT_D = 64;                  // head size
constexpr int AT_ROWS = 128;              // query rows per CTA (UMMA M)
constexpr int AT_KEYS = 64;               // keys per tile (UMMA N of S, K of P V)
constexpr int AT_THREADS = 288;           // 4 staging warps, 4 softmax warps, 1 MMA warp
constexpr int AT_STAGES = 3;              // key / value tiles in flight
constexpr int AT_KV_BYTES = AT_KEYS * AT_D * 2;
constexpr int AT_Q_BYTES = AT_ROWS * AT_D * 2;
constexpr int AT_P_BYTES = AT_ROWS * AT_KEYS * 2;
constexpr int AT_SPLIT_TILES = 8;         // key tiles a CTA should have before a tile's keys are shared out
constexpr float AT_LAZY = 8.0f;           // log2 of how far a probability may exceed 1 before a rescale
constexpr long long AT_WAIT_CYCLES = 2000000000LL;

__device__ int g_at_error = 0;

__device__ __forceinline__ bool at_wait(uint32_t bar, uint32_t parity, int where) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long start = clock64();
    int it = 0;
    while (!mbar_try_wait(bar, parity)) {
        if ((++it & 255) == 0) {
            if (*(volatile int*)&g_at_error != 0) return false;
            if (clock64() - start > AT_WAIT_CYCLES) {
                atomicCAS(&g_at_error, 0, where);
                return false;
            }
        }
    }
    return true;
}

__device__ __forceinline__ uint32_t pack_bf16_pair(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// Packed 32-bit arithmetic (two lanes per instruction): the softmax threads are bound by the
// number of instructions they issue, and most of them are elementwise on pairs.
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) { return __ffma2_rn(a, b, c); }
__device__ __forceinline__ float2 add2(float2 a, float2 b) { return __fadd2_rn(a, b); }

__device__ __forceinline__ float fmax3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}

__device__ __forceinline__ void stsm_x4(uint32_t addr, const uint32_t (&r)[4]) {
    asm volatile("stmatrix.sync.aligned.m8n8.x4.shared.b16 [%0], {%1,%2,%3,%4};\n" ::"r"(addr), "r"(r[0]),
                 "r"(r[1]), "r"(r[2]), "r"(r[3])
                 : "memory");
}

__global__ void __launch_bounds__(AT_THREADS, 2)
attn_prefill_tc_kernel(const __nv_bfloat16* q, const __nv_bfloat16* pool, __nv_bfloat16* out,
                       const int* positions, const int* tok_seq, const int* block_table, int bt_stride,
                       const int* tile_tok0, const int* tile_ntok, int H, int Hkv, int P, int window,
                       float scale, int p_shift, const __nv_bfloat16* gate, int64_t ldg, int max_split,
                       float* part_o, float* part_ml, int* tickets) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    __shared__ int s_last;
    pdl_launch_dependents();
    pdl_wait();
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t q_tile = base;
    const uint32_t k_tile0 = q_tile + AT_Q_BYTES;                         // AT_STAGES stages
    const uint32_t vt_tile0 = k_tile0 + AT_STAGES * AT_KV_BYTES;          // [d][key]
    const uint32_t v_stage = vt_tile0 + AT_STAGES * AT_KV_BYTES;          // [key][d] as it lands (one tile)
    const uint32_t p_tile0 = v_stage + AT_KV_BYTES;                       // two P tiles, used in turn
    const uint32_t bars = p_tile0 + 2 * AT_P_BYTES;
    auto kv_full = [&](int s) { return bars + (uint32_t)s * 8; };
    auto kv_empty = [&](int s) { return bars + (uint32_t)(AT_STAGES + s) * 8; };
    auto s_full = [&](int b) { return bars + (uint32_t)(2 * AT_STAGES + b) * 8; };
    auto s_free = [&](int b) { return bars + (uint32_t)(2 * AT_STAGES + 2 + b) * 8; };
    const uint32_t p_full = bars + (2 * AT_STAGES + 4) * 8, pv_full = p_full + 8;
    const uint32_t tmem_slot = p_full + 24;
    volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(smem_raw + (tmem_slot - smem_u32(smem_raw)));

    const int G = H / Hkv;
    // the grid is one-dimensional with the KV head fastest and the tiles in reverse: a causal
    // tile late in its sequence reads the most keys, so the longest CTAs start first
    const int kvh = blockIdx.x % Hkv;
    const int tile = gridDim.x / Hkv - 1 - blockIdx.x / Hkv;
    const int tok0 = tile_tok0[tile], ntok = tile_ntok[tile];
    if (ntok <= 0) return;       // an unused entry of a fixed-length tile list (captured steps)
    const int rows = ntok * G;
    const int seq = tok_seq[tok0];
    const int* bt_row = block_table + (size_t)seq * bt_stride;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int pos_first = positions[tok0];
    const int pos_last = pos_first + ntok - 1;       // consecutive positions within a tile
    const int lo = window > 0 ? max(0, pos_first - window + 1) : 0;
    const int j_begin = (lo / AT_KEYS) * AT_KEYS;
    // Up to `max_split` CTAs (blockIdx.y) share a tile's keys, as many as leave each at least
    // AT_SPLIT_TILES key tiles: CTA `split` takes key tiles split, split + nsplit, ...; the ones
    // beyond that number have nothing to do. (The launch fixes the most; the tile decides.)
    const int split = blockIdx.y;
    const int all_tiles = (pos_last - j_begin) / AT_KEYS + 1;
    const int nsplit = min(max_split, max(1, all_tiles / AT_SPLIT_TILES));
    if (split >= nsplit) return;
    const int n_tiles = (all_tiles - split + nsplit - 1) / nsplit;       // at least one
    auto tile_j0 = [&](int it) { return j_begin + (split + it * nsplit) * AT_KEYS; };

    if (tid == 0) {
        for (int i = 0; i < AT_STAGES; ++i) {
            mbar_init(kv_full(i), 1);
            mbar_init(kv_empty(i), 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(s_full(i), 1);
            mbar_init(s_free(i), 4);
        }
        mbar_init(p_full, 1);
        mbar_init(pv_full, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 8) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot), "r"(256u)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = *tmem_slot_ptr;
    const uint32_t tmem_pv = tmem + 2 * AT_KEYS;         // columns [128, 192); S_b at [64 b, 64 b + 64)

    // The register file is shared unevenly: the staging warps give registers up and the softmax
    // warps (a whole row of scores each) take them.
    if (warp < 4) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 64;");
        // ---- staging ----
        PagedLoader<AT_D, AT_KEYS, 128> loader;
        loader.init(tid, kvh, Hkv, P, p_shift);
        // Q: row r = token * G + head; rows past the tile are zero
        for (int i = tid; i < AT_ROWS * (AT_D / 8); i += 128) {
            const int r = i >> 3, c = i & 7;
            const bool valid = r < rows;
            const __nv_bfloat16* src = q;
            if (valid) src = q + ((size_t)(tok0 + r / G) * H + kvh * G + r % G) * AT_D + c * 8;
            cp_async16(q_tile + tile_off<AT_D>(r, c), src, valid);
        }
        // One copy is in flight while the tile before it is turned and handed over. The copy of
        // tile it + 1 needs the stage that tile it - 2 held, which P V of that tile gives back a
        // whole softmax pass before S of tile it + 1 is wanted; looking two tiles ahead instead
        // made this warp group wait for the stage of tile it - 1 with tile it + 1 lying unturned,
        // and the softmax threads waited for S every tile. The block-table entries of a tile are
        // fetched one tile ahead of its copies.
        bool ok = true;
        auto issue = [&](int it) {
            const int s = it % AT_STAGES;
            if (it >= AT_STAGES && ok) ok = at_wait(kv_empty(s), (uint32_t)((it / AT_STAGES - 1) & 1), 1);
            const int j0 = tile_j0(it);
            const uint32_t kt = k_tile0 + (uint32_t)s * AT_KV_BYTES, vs = v_stage;
            if (p_shift >= 0) {
                loader.issue_looked_up(kt, vs, pool, j0, lo, pos_last);
                if (it + 1 < n_tiles) loader.lookup(bt_row, tile_j0(it + 1), lo, pos_last);
            } else {
                load_tile<AT_D>(kt, pool, bt_row, j0, AT_KEYS, lo, pos_last, kvh, Hkv, P, 0, tid, 128);
                load_tile<AT_D>(vs, pool, bt_row, j0, AT_KEYS, lo, pos_last, kvh, Hkv, P, 1, tid, 128);
            }
            cp_async_commit();
        };
        if (p_shift >= 0 && n_tiles > 0) loader.lookup(bt_row, tile_j0(0), lo, pos_last);
        if (n_tiles > 0) issue(0);
        // (after a failed wait the loop still runs to its end, without waiting: every thread must
        // meet every named barrier)
        for (int it = 0; it < n_tiles; ++it) {
            const int s = it % AT_STAGES;
            cp_async_wait<0>();
            asm volatile("bar.sync 2, 128;" ::: "memory");
            // V [key][d] -> [d][key]: 64 blocks of 8 x 8, four per instruction pair, sixteen pairs
            const uint32_t vs = v_stage, vt = vt_tile0 + (uint32_t)s * AT_KV_BYTES;
            const int m = lane >> 3, i8 = lane & 7;
#pragma unroll
            for (int o = 0; o < 4; ++o) {
                const int b = (warp * 4 + o) * 4 + m;            // this lane's block: key block, d chunk
                const int kb = b >> 3, c = b & 7;
                uint32_t r4[4];
                ldsm_x4_trans(r4, vs + tile_off<AT_D>(kb * 8 + i8, c));
                stsm_x4(vt + tile_off<AT_D>(c * 8 + i8, kb), r4);
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            asm volatile("bar.sync 2, 128;" ::: "memory");
            if (tid == 0) mbar_arrive(kv_full(s));
            if (it + 1 < n_tiles) issue(it + 1);
        }
    } else if (warp == 8) {
        // ---- MMA issuer ----
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc(AT_KEYS);      // 128 x 64, both products
            const uint64_t qdesc = umma_desc(q_tile);
            bool ok = true;
            auto issue_s = [&](int j) {
                const int s = j % AT_STAGES, b = j & 1;
                ok = ok && at_wait(kv_full(s), (uint32_t)((j / AT_STAGES) & 1), 2);
                if (ok && j >= 2) ok = at_wait(s_free(b), (uint32_t)(((j >> 1) - 1) & 1), 3);
                if (!ok) return;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint64_t kdesc = umma_desc(k_tile0 + (uint32_t)s * AT_KV_BYTES);
#pragma unroll
                for (int k = 0; k < AT_D / 16; ++k)
                    umma_bf16(tmem + (uint32_t)b * AT_KEYS, qdesc + 2 * k, kdesc + 2 * k, idesc, k > 0 ? 1u : 0u);
                umma_commit(s_full(b));
            };
            if (n_tiles > 0) issue_s(0);
            for (int j = 0; j < n_tiles && ok; ++j) {
                if (j + 1 < n_tiles) issue_s(j + 1);
                if (!ok) break;
                ok = at_wait(p_full, (uint32_t)(j & 1), 4);    // P_j written, the output rescaled if need be
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const int s = j % AT_STAGES;
                const uint64_t vdesc = umma_desc(vt_tile0 + (uint32_t)s * AT_KV_BYTES);
                const uint64_t pdesc = umma_desc(p_tile0 + (uint32_t)(j & 1) * AT_P_BYTES);
#pragma unroll
                for (int k = 0; k < AT_KEYS / 16; ++k)
                    umma_bf16(tmem_pv, pdesc + 2 * k, vdesc + 2 * k, idesc, (j > 0 || k > 0) ? 1u : 0u);
                umma_commit(pv_full);
                umma_commit(kv_empty(s));
            }
        }
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 128;");
        // ---- softmax: thread r owns query row r ----
        // The output accumulates in tensor memory over all key tiles (P V with the accumulate
        // flag) under a reference maximum m_ref that follows the true maximum lazily: it is
        // raised, and the accumulated row and sum rescaled, only when some row of the warp sees a
        // score more than AT_LAZY (in log2 units) above it. Until then probabilities may exceed 1,
        // by at most 2^AT_LAZY; in 32-bit accumulation, with the division by the row sum at the
        // end, that changes nothing but the scale the intermediate values live at.
        const int r = tid - 128;
        const int quarter = warp & 3;
        const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
        const int pos_r = r < rows ? pos_first + r / G : -1;
        const int lo_r = window > 0 ? pos_r - window + 1 : 0;
        const float scale_log2 = scale * LOG2E;
        float m_ref = -INFINITY;
        float2 l_run = make_float2(0.f, 0.f), l_alt = make_float2(0.f, 0.f);   // the row sum in four lanes
        bool ok = true;
        for (int j = 0; j < n_tiles; ++j) {
            const int b = j & 1, j0 = tile_j0(j);
            // (after a failed wait the loop still runs to its end, without waiting: every thread
            // must meet every named barrier)
            if (ok) ok = at_wait(s_full(b), (uint32_t)((j >> 1) & 1), 6);
            ok = __all_sync(0xffffffffu, ok);
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t s_addr = tmem + lane_base + (uint32_t)b * AT_KEYS;
            float s_lo[32], s_hi[32];                    // the row's 64 scores stay in registers
            tmem_ld32(s_addr, s_lo);
            tmem_ld32(s_addr + 32u, s_hi);
            // S_b is read: the MMA warp may overwrite it with the tile after next
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(s_free(b));
            // a tile every row of the CTA sees whole needs no comparisons
            const bool masked = j0 + AT_KEYS - 1 > pos_first || (window > 0 && j0 < pos_last - window + 1) ||
                                rows < AT_ROWS;
            // the row's maximum over the tile's visible keys (the scale is positive)
            // (four chains: a thread has few other warps to hide a 64-deep dependency behind)
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
            if (masked) {
#pragma unroll
                for (int e = 0; e < 32; ++e) {
                    const int key = j0 + e;
                    if (key <= pos_r && key >= lo_r) mx4[e & 1] = fmaxf(mx4[e & 1], s_lo[e]);
                    if (key + 32 <= pos_r && key + 32 >= lo_r) mx4[2 + (e & 1)] = fmaxf(mx4[2 + (e & 1)], s_hi[e]);
                }
            } else {
#pragma unroll
                for (int e = 0; e < 32; ++e) mx4[e & 3] = fmax3(mx4[e & 3], s_lo[e], s_hi[e]);
            }
            const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * scale_log2;
            const bool raise = __any_sync(0xffffffffu, mx > m_ref + AT_LAZY);
            if (raise) {
                const float m_new = fmaxf(m_ref, mx);
                if (j >= 1) {
                    // the product of the tile before must have landed before the output is touched
                    if (ok) ok = at_wait(pv_full, (uint32_t)((j - 1) & 1), 7);
                    ok = __all_sync(0xffffffffu, ok);
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const float alpha = m_new == -INFINITY ? 1.0f : fast_exp2(m_ref - m_new);
#pragma unroll
                    for (int c = 0; c < AT_D; c += 16) {          // (narrow: the scores stay in registers)
                        float part[16];
                        tmem_ld16(tmem_pv + lane_base + (uint32_t)c, part);
#pragma unroll
                        for (int e = 0; e < 16; ++e) part[e] *= alpha;
                        tmem_st16(tmem_pv + lane_base + (uint32_t)c, part);
                    }
                    l_run.x *= alpha;
                    l_run.y *= alpha;
                    l_alt.x *= alpha;
                    l_alt.y *= alpha;
                }
                m_ref = m_new;
            }
            const float neg_m = m_ref == -INFINITY ? 0.f : -m_ref;
            // probabilities, rounded to bfloat16 into the A operand of P V
            // (P_j goes to the tile that P_{j-2} used: S_j is complete, and the tensor pipe runs
            // in order, so the product that read P_{j-2} is complete too)
            const uint32_t p_tile = p_tile0 + (uint32_t)(j & 1) * AT_P_BYTES;
            auto emit = [&](const float (&part)[32], int c) {
                uint32_t packed[16];
                if (masked) {
#pragma unroll
                    for (int e = 0; e < 32; e += 2) {
                        float p0 = 0.f, p1 = 0.f;
                        const int key = j0 + c + e;
                        if (key <= pos_r && key >= lo_r) p0 = fast_exp2(fmaf(part[e], scale_log2, neg_m));
                        if (key + 1 <= pos_r && key + 1 >= lo_r) p1 = fast_exp2(fmaf(part[e + 1], scale_log2, neg_m));
                        if (e & 2) l_alt = add2(l_alt, make_float2(p0, p1));
                        else l_run = add2(l_run, make_float2(p0, p1));
                        packed[e >> 1] = pack_bf16_pair(p0, p1);
                    }
                } else {
                    const float2 sc2 = make_float2(scale_log2, scale_log2), nm2 = make_float2(neg_m, neg_m);
#pragma unroll
                    for (int e = 0; e < 32; e += 2) {
                        const float2 x = fma2(make_float2(part[e], part[e + 1]), sc2, nm2);
                        const float2 pp = make_float2(fast_exp2(x.x), fast_exp2(x.y));
                        if (e & 2) l_alt = add2(l_alt, pp);
                        else l_run = add2(l_run, pp);
                        packed[e >> 1] = pack_bf16_pair(pp.x, pp.y);
                    }
                }
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const uint32_t at = p_tile + tile_off<AT_D>(r, (c >> 3) + k);
                    asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(at), "r"(packed[4 * k]),
                                 "r"(packed[4 * k + 1]), "r"(packed[4 * k + 2]), "r"(packed[4 * k + 3])
                                 : "memory");
                }
            };
            emit(s_lo, 0);
            emit(s_hi, 32);
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            asm volatile("bar.sync 3, 128;" ::: "memory");
            if (r == 0) mbar_arrive(p_full);
        }
        if (ok && n_tiles > 0) {
            ok = at_wait(pv_full, (uint32_t)((n_tiles - 1) & 1), 8);
            ok = __all_sync(0xffffffffu, ok);
        }
        if (ok) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const float l_row = (l_run.x + l_run.y) + (l_alt.x + l_alt.y);
            __nv_bfloat16* dst = r < rows ? out + ((size_t)(tok0 + r / G) * H + kvh * G + r % G) * AT_D : nullptr;
            // the per-head output gate, if the layer has one: round(round(o) * round(sigmoid(g)))
            float gs = 1.0f;
            if (gate != nullptr && dst != nullptr) {
                const float gv = __bfloat162float(gate[(size_t)(tok0 + r / G) * ldg + kvh * G + r % G]);
                gs = round_as<__nv_bfloat16>(1.0f / (1.0f + expf(-gv)));
            }
            // 16 finished values of the row: normalised, rounded, gated, stored
            auto store16 = [&](int c, const float (&part)[16], float inv) {
                if (dst == nullptr) return;
                uint32_t packed[8];
#pragma unroll
                for (int e = 0; e < 16; e += 2) {
                    packed[e >> 1] = pack_bf16_pair(part[e] * inv, part[e + 1] * inv);
                    if (gate != nullptr) {
                        const float2 f = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&packed[e >> 1]));
                        packed[e >> 1] = pack_bf16_pair(f.x * gs, f.y * gs);
                    }
                }
                *reinterpret_cast<uint4*>(dst + c) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
                *reinterpret_cast<uint4*>(dst + c + 8) = make_uint4(packed[4], packed[5], packed[6], packed[7]);
            };
            if (nsplit == 1) {
                const float inv = l_row > 0.f ? 1.0f / l_row : 0.f;
#pragma unroll
                for (int c = 0; c < AT_D; c += 16) {
                    float part[16];
                    tmem_ld16(tmem_pv + lane_base + (uint32_t)c, part);
                    store16(c, part, inv);
                }
            } else {
                // This CTA's share of the keys: the unnormalised row, its reference maximum and its
                // sum go to scratch memory ([column][row], so that the 128 rows' accesses are
                // contiguous); the CTA of this (tile, KV head) that draws the last ticket merges.
                const size_t group = (size_t)tile * Hkv + kvh;
                const size_t slot = group * max_split + split;
                float* po = part_o + slot * (size_t)(AT_ROWS * AT_D);
                if (n_tiles > 0) {
#pragma unroll
                    for (int c = 0; c < AT_D; c += 16) {
                        float part[16];
                        tmem_ld16(tmem_pv + lane_base + (uint32_t)c, part);
#pragma unroll
                        for (int e = 0; e < 16; ++e) po[(size_t)(c + e) * AT_ROWS + r] = part[e];
                    }
                }
                part_ml[(slot * AT_ROWS + r) * 2] = n_tiles > 0 ? m_ref : -INFINITY;
                part_ml[(slot * AT_ROWS + r) * 2 + 1] = l_row;
                __threadfence();
                asm volatile("bar.sync 3, 128;" ::: "memory");
                if (r == 0) s_last = atomicAdd(&tickets[group], 1) == nsplit - 1;
                asm volatile("bar.sync 3, 128;" ::: "memory");
                if (s_last) {
                    __threadfence();
                    const float* ml = part_ml + group * max_split * (size_t)(AT_ROWS * 2);
                    float M = -INFINITY;
                    for (int sp = 0; sp < nsplit; ++sp) M = fmaxf(M, __ldcg(&ml[((size_t)sp * AT_ROWS + r) * 2]));
                    float L = 0.f;
                    float acc[AT_D];
#pragma unroll
                    for (int c = 0; c < AT_D; ++c) acc[c] = 0.f;
                    for (int sp = 0; sp < nsplit; ++sp) {
                        const float ms = __ldcg(&ml[((size_t)sp * AT_ROWS + r) * 2]);
                        if (ms == -INFINITY) continue;         // nothing visible in that share: its row was not written
                        const float f = fast_exp2(ms - M);
                        L += __ldcg(&ml[((size_t)sp * AT_ROWS + r) * 2 + 1]) * f;
                        const float* src = part_o + (group * max_split + sp) * (size_t)(AT_ROWS * AT_D) + r;
#pragma unroll
                        for (int c = 0; c < AT_D; ++c) acc[c] = fmaf(__ldcg(src + (size_t)c * AT_ROWS), f, acc[c]);
                    }
                    const float inv = L > 0.f ? 1.0f / L : 0.f;
#pragma unroll
                    for (int c = 0; c < AT_D; c += 16) {
                        float part[16];
#pragma unroll
                        for (int e = 0; e < 16; ++e) part[e] = acc[c + e];
                        store16(c, part, inv);
                    }
                    if (r == 0) tickets[group] = 0;
                }
            }
        }
    }
    // ---- teardown: the tensor memory goes back whatever happened above ----
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 8) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(256u) : "memory");
    }
}

}  // namespace

// Whether the tcgen05 prefill kernel takes this shape: head size 64, a group that divides 128.
TK_API int tk_attn_prefill_tc_supported(int H, int Hkv, int D) {
    if (Hkv <= 0 || H % Hkv || D != AT_D) return 0;
    const int G = H / Hkv;
    return G >= 1 && G <= AT_ROWS && AT_ROWS % G == 0;
}

// Tokens of one sequence that a tile of this kernel holds (what the caller cuts portions into).
TK_API int tk_attn_prefill_tc_tokens(int H, int Hkv) { return AT_ROWS / (H / Hkv); }

// Floats of scratch for n_tiles tiles split nsplit ways (nothing unsplit): the unnormalised rows
// [n_tiles, Hkv, nsplit, 64, 128], then each row's reference maximum and sum [.., 128, 2].
TK_API int64_t tk_attn_prefill_tc_scratch(int n_tiles, int Hkv, int nsplit) {
    return nsplit <= 1 ? 0 : (int64_t)n_tiles * Hkv * nsplit * (AT_ROWS * AT_D + AT_ROWS * 2);
}

// 0, or where a CTA gave up waiting on a barrier since the last call (1 staging, 2-4 MMA issuer,
// 6-8 softmax). Resets the word.
TK_API int tk_attn_prefill_tc_status() {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_at_error, sizeof(int)) != cudaSuccess) return -1;
    if (v != 0) cudaMemcpyToSymbol(g_at_error, &zero, sizeof(int));
    return v;
}

// q: [T, H, 64] bfloat16; kv_pool: [pages, 2, Hkv, P, 64]; out: [T, H, 64]; tiles of at most
// tk_attn_prefill_tc_tokens tokens of one sequence with consecutive positions; window 0 = none.
// gate: [T, >= H] bfloat16 with rows ldg apart, the per-head output gate applied to what is
// written (null: none). nsplit > 1: up to that many CTAs share a tile's keys (alternate key tiles;
// each tile takes as many as leave a CTA 8 key tiles), for steps with few tiles and long
// contexts, where one CTA per tile would walk its keys alone on an idle GPU; `scratch`: tk_attn_prefill_tc_scratch floats, `tickets`: n_tiles * Hkv ints that are
// zero and are zero again afterwards (the last CTA of a tile to finish merges the shares).
TK_API int tk_attn_prefill_tc(const void* q, const void* kv_pool, void* out, const int* positions,
                              const int* tok_seq, const int* block_table, int bt_stride,
                              const int* tile_tok0, const int* tile_ntok, int n_tiles, int H, int Hkv, int D,
                              int P, int window, float scale, const void* gate, int64_t ldg, int nsplit,
                              float* scratch, int* tickets, cudaStream_t stream) {
    TK_CHECK_ARG(tk_attn_prefill_tc_supported(H, Hkv, D), "attn_prefill_tc: shape H=%d Hkv=%d D=%d is not taken "
                 "(head size 64, a group that divides 128)", H, Hkv, D);
    TK_CHECK_ARG(P > 0 && n_tiles >= 0, "attn_prefill_tc: bad page size or tile count");
    TK_CHECK_ARG(nsplit >= 1 && nsplit <= 64 && (nsplit == 1 || (scratch != nullptr && tickets != nullptr)),
                 "attn_prefill_tc: %d splits (1..64; more than one needs scratch memory and tickets)", nsplit);
    if (n_tiles == 0) return 0;
    float* part_o = scratch;
    float* part_ml = scratch ? scratch + (size_t)n_tiles * Hkv * nsplit * (AT_ROWS * AT_D) : nullptr;
    int shift = -1;
    if ((P & (P - 1)) == 0) {
        shift = 0;
        while ((1 << shift) < P) ++shift;
    }
    const size_t smem = 1024 + AT_Q_BYTES + (2 * AT_STAGES + 1) * AT_KV_BYTES + 2 * AT_P_BYTES + (2 * AT_STAGES + 8) * 8 + 64;
    cudaError_t e = cudaFuncSetAttribute(attn_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess)
        e = tk_launch(attn_prefill_tc_kernel, dim3(n_tiles * Hkv, nsplit), dim3(AT_THREADS), smem, stream,
                      (const __nv_bfloat16*)q, (const __nv_bfloat16*)kv_pool, (__nv_bfloat16*)out, positions, tok_seq,
                      block_table, bt_stride, tile_tok0, tile_ntok, H, Hkv, P, window, scale, shift,
                      (const __nv_bfloat16*)gate, ldg, nsplit, part_o, part_ml, tickets);
    if (e != cudaSuccess) {
        tk_set_error("attn_prefill_tc: launch failed: %s", cudaGetErrorString(e));
        cudaGetLastError();
        return -2;
    }
    return 0;
}
