// Tensor-core matrix product for sm_100a: TMA (cp.async.bulk.tensor) stages both operands in
// shared memory behind mbarriers, one thread issues tcgen05.mma (UMMA, 128 x BN x 16, bfloat16 in,
// 32-bit accumulator in tensor memory), four warps read the accumulator back with tcgen05.ld for
// the epilogue.
//
//   D[i, j] = sum_k A[i, k] * B[j, k]        A: [rows_a, K], B: [rows_b, K], both K-major bf16
//
// Decode ("weights as A"): A = W [N, K], B = x [tokens, K]; the 128-row MMA tile is filled with
// weight rows and the few tokens are the MMA's N (16..256), so no tensor-core row is wasted on
// padding the batch; D is stored transposed into out[token, n]. Matrices with few rows are split
// along K over the CTAs of a thread-block cluster (up to 8); every CTA leaves its partial tile in
// its own shared memory and each sums a share of the rows over all of them through distributed
// shared memory, so one kernel does it all without scratch memory or atomics.
// Prefill ("tokens as A"): A = x, B = W, D is stored as it is.
//
// Warp roles in a CTA of 192 threads: warp 0 produces (one lane issues TMA), warp 1 allocates
// tensor memory and issues the MMAs, warps 2..5 are the epilogue (warp w may touch TMEM lanes
// 32 (w % 4) .. +31). In decode the weight tiles of the first stages are requested before
// griddepcontrol.wait: they stream while the kernel that produces x is still running.
//
// Every wait on an mbarrier is bounded: after about a second the kernel records where it gave
// up in an error word, skips the rest of its work, frees its tensor memory and returns; the
// host reads the word through tk_gemm_tc_status().
#include <cooperative_groups.h>

#include "tcgen05.cuh"

namespace cg = cooperative_groups;

namespace {

constexpr int BM = 128;          // rows of A per tile (UMMA M)
constexpr int BK = 64;           // K elements per stage: 128 bytes, one swizzle atom wide
constexpr int TC_THREADS = 192;
constexpr int A_TILE_BYTES = BM * BK * 2;

__device__ int g_tc_error = 0;

// Bounded wait: false (and an error code recorded) if the phase did not complete in ~1 s.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int where) {
    const long long start = clock64();
    while (!mbar_try_wait(bar, parity)) {
        if (clock64() - start > 2000000000LL) {
            atomicCAS(&g_tc_error, 0, where);
            return false;
        }
    }
    return true;
}

__device__ __forceinline__ void epi_bar_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

// TRANSPOSED: D[i, j] -> out[j, i] (decode, weights as A); otherwise out[i, j] (tokens as A).
// SWIGLU (decode only): rows of A come in blocks of 16, 8 gate rows then the 8 up rows of the
// same channels; out[j, c] = silu(gate) * up, out width rows_a / 2.
template <int BN, bool TRANSPOSED, bool SWIGLU, typename TO>
__global__ void __launch_bounds__(TC_THREADS)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
               TO* out, int64_t ldo, const float* __restrict__ bias, int rows_a, int rows_b, int K,
               int stages, int splitk, int cluster_k) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    constexpr int B_TILE_BYTES = BN * BK * 2;
    constexpr int STAGE_BYTES = A_TILE_BYTES + B_TILE_BYTES;
    constexpr int TMEM_COLS = BN < 32 ? 32 : BN;
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t bars = smem_base + (uint32_t)stages * STAGE_BYTES;   // full[s], empty[s], tmem_full
    const uint32_t tmem_slot = bars + (2 * stages + 1) * 8;
    auto full_bar = [&](int s) { return bars + (uint32_t)s * 8; };
    auto empty_bar = [&](int s) { return bars + (uint32_t)(stages + s) * 8; };
    const uint32_t tmem_full_bar = bars + (uint32_t)(2 * stages) * 8;
    volatile uint32_t* tmem_slot_ptr =
        reinterpret_cast<volatile uint32_t*>(smem_raw + (tmem_slot - smem_u32(smem_raw)));

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int a_row0 = blockIdx.x * BM, b_row0 = blockIdx.y * BN;
    const int kb_total = (K + BK - 1) / BK;
    const int kb_per = (kb_total + splitk - 1) / splitk;
    const int kb_begin = blockIdx.z * kb_per;
    const int kb_end = min(kb_total, kb_begin + kb_per);
    const int n_kb = max(0, kb_end - kb_begin);

    pdl_launch_dependents();
    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        mbar_init(tmem_full_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot),
                     "r"((uint32_t)TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_d = *tmem_slot_ptr;
    bool ok = true;

    if (warp == 0) {
        // ---- producer ----
        if (lane == 0 && n_kb > 0) {
            int first = 0;
            if (TRANSPOSED) {
                // weights first: they do not depend on the kernel before this one
                first = min(stages, n_kb);
                for (int i = 0; i < first; ++i) {
                    mbar_expect_tx(full_bar(i), STAGE_BYTES);
                    tma_load_2d(smem_base + (uint32_t)i * STAGE_BYTES, &tmap_a, (kb_begin + i) * BK, a_row0,
                                full_bar(i));
                }
                pdl_wait();
                for (int i = 0; i < first; ++i)
                    tma_load_2d(smem_base + (uint32_t)i * STAGE_BYTES + A_TILE_BYTES, &tmap_b,
                                (kb_begin + i) * BK, b_row0, full_bar(i));
            } else {
                pdl_wait();
            }
            for (int i = first; i < n_kb && ok; ++i) {
                const int s = i % stages;
                const uint32_t parity = ((i / stages) & 1) ^ 1;
                ok = mbar_wait(empty_bar(s), parity, 1);
                if (!ok) break;
                mbar_expect_tx(full_bar(s), STAGE_BYTES);
                const uint32_t dst = smem_base + (uint32_t)s * STAGE_BYTES;
                tma_load_2d(dst, &tmap_a, (kb_begin + i) * BK, a_row0, full_bar(s));
                tma_load_2d(dst + A_TILE_BYTES, &tmap_b, (kb_begin + i) * BK, b_row0, full_bar(s));
            }
        } else if (lane == 0) {
            pdl_wait();
        }
    } else if (warp == 1) {
        // ---- MMA issuer ----
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc(BN);
            for (int i = 0; i < n_kb && ok; ++i) {
                const int s = i % stages;
                ok = mbar_wait(full_bar(s), (i / stages) & 1, 2);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t a_addr = smem_base + (uint32_t)s * STAGE_BYTES;
                const uint64_t adesc = umma_desc(a_addr), bdesc = umma_desc(a_addr + A_TILE_BYTES);
#pragma unroll
                for (int k = 0; k < BK / 16; ++k)     // 32 bytes further along K per step
                    umma_bf16(tmem_d, adesc + 2 * k, bdesc + 2 * k, idesc, (i > 0 || k > 0) ? 1u : 0u);
                umma_commit(empty_bar(s));            // the stage is free once these MMAs are done
            }
            umma_commit(tmem_full_bar);
        }
    } else {
        // ---- epilogue: warps 2..5, TMEM lanes 32 (warp % 4) .. +31 ----
        pdl_wait();
        const int lane_group = warp & 3;
        const int epi_tid = (warp - 2) * 32 + lane;
        ok = n_kb > 0 ? mbar_wait(tmem_full_bar, 0, 3) : true;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const int i_row = a_row0 + lane_group * 32 + lane;          // row of A / D
        const bool row_ok = i_row < rows_a;
        float bias_i = 0.f;
        if (TRANSPOSED && bias != nullptr && row_ok) bias_i = bias[i_row];
        // columns c .. c + 15 of this thread's row, finished: bias, activation, store
        auto finalize = [&](int c, float (&part)[16]) {
            if (TRANSPOSED && SWIGLU) {
                const bool is_gate = (i_row & 15) < 8;
#pragma unroll
                for (int e = 0; e < 16; ++e) {
                    const float mine = round_as<TO>(part[e] + bias_i);
                    const float other = __shfl_xor_sync(0xffffffffu, mine, 8);       // gate <-> up
                    const int jj = b_row0 + c + e;
                    if (is_gate && row_ok && i_row + 8 < rows_a && jj < rows_b) {
                        const float act = silu_as<TO>(mine);
                        out[(size_t)jj * ldo + (i_row >> 4) * 8 + (i_row & 7)] = from_f<TO>(act * other);
                    }
                }
            } else if (TRANSPOSED) {
#pragma unroll
                for (int e = 0; e < 16; ++e) {
                    const int jj = b_row0 + c + e;
                    if (row_ok && jj < rows_b) out[(size_t)jj * ldo + i_row] = from_f<TO>(part[e] + bias_i);
                }
            } else {
#pragma unroll
                for (int e = 0; e < 16; ++e) {
                    const int jj = b_row0 + c + e;
                    if (row_ok && jj < rows_b)
                        out[(size_t)i_row * ldo + jj] = from_f<TO>(part[e] + (bias != nullptr ? bias[jj] : 0.f));
                }
            }
        };
        const bool have = ok && n_kb > 0;
        if (cluster_k > 1) {
            // split K over a cluster: this CTA's partial tile goes to its own shared memory
            // (the pipeline stages are done with: every MMA that read them has completed)
            float* mine = reinterpret_cast<float*>(smem_raw + (smem_base - smem_u32(smem_raw)));
            const int row_local = lane_group * 32 + lane;
            for (int c = 0; c < BN; c += 16) {
                float part[16];
                if (have) {
                    tmem_ld16(tmem_d + ((uint32_t)(lane_group * 32) << 16) + (uint32_t)c, part);
                } else {
#pragma unroll
                    for (int e = 0; e < 16; ++e) part[e] = 0.f;
                }
#pragma unroll
                for (int e = 0; e < 16; ++e) mine[(c + e) * BM + row_local] = part[e];
            }
        } else {
            for (int c = 0; c < BN; c += 16) {
                float part[16];
                if (have) {
                    tmem_ld16(tmem_d + ((uint32_t)(lane_group * 32) << 16) + (uint32_t)c, part);
                    finalize(c, part);
                }
            }
        }
    }
    if (cluster_k > 1) {
        // every CTA of the cluster holds a partial [BN][128] tile; rank r sums rows
        // [r * 128 / k, (r + 1) * 128 / k) over all ranks through distributed shared memory
        cg::cluster_group cluster = cg::this_cluster();
        cluster.sync();
        if (warp >= 2) {
            float* mine = reinterpret_cast<float*>(smem_raw + (smem_base - smem_u32(smem_raw)));
            const int share = BM / cluster_k;
            const int row_begin = (int)cluster.block_rank() * share;
            const int epi_tid = (warp - 2) * 32 + lane;
            // four consecutive rows of one column, summed over the ranks: the remote loads of a
            // thread are independent 16-byte reads, all in flight together
            auto total4 = [&](int row, int col, float (&v)[4]) {
                float4 part[8];
#pragma unroll
                for (int r = 0; r < 8; ++r)
                    if (r < cluster_k)
                        part[r] = *reinterpret_cast<const float4*>(cluster.map_shared_rank(mine, r) + col * BM + row);
                v[0] = v[1] = v[2] = v[3] = 0.f;
#pragma unroll
                for (int r = 0; r < 8; ++r)
                    if (r < cluster_k) {
                        v[0] += part[r].x;
                        v[1] += part[r].y;
                        v[2] += part[r].z;
                        v[3] += part[r].w;
                    }
            };
            // four consecutive elements of a row of `out`
            auto store4 = [&](TO* dst, const float (&v)[4], int n_ok) {
                if (n_ok == 4 && ((uintptr_t)dst % (4 * sizeof(TO))) == 0) {
                    if constexpr (sizeof(TO) == 2) {
                        __nv_bfloat162 lo = __floats2bfloat162_rn(v[0], v[1]), hi = __floats2bfloat162_rn(v[2], v[3]);
                        uint2 raw;
                        raw.x = *reinterpret_cast<uint32_t*>(&lo);
                        raw.y = *reinterpret_cast<uint32_t*>(&hi);
                        *reinterpret_cast<uint2*>(dst) = raw;
                    } else {
                        *reinterpret_cast<float4*>(dst) = make_float4(v[0], v[1], v[2], v[3]);
                    }
                } else {
                    for (int e = 0; e < n_ok; ++e) dst[e] = from_f<TO>(v[e]);
                }
            };
            if (TRANSPOSED && SWIGLU) {
                const int groups = share / 8;              // runs of 4 gate rows in the share
                for (int idx = epi_tid; idx < groups * BN; idx += 128) {
                    const int col = idx / groups, g = idx % groups;
                    const int row = row_begin + (g >> 1) * 16 + (g & 1) * 4;
                    const int i_row = a_row0 + row, jj = b_row0 + col;
                    if (i_row + 8 < rows_a && jj < rows_b) {
                        float gate[4], up[4], res[4];
                        total4(row, col, gate);
                        total4(row + 8, col, up);
                        int n_ok = 0;
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            if (i_row + e + 8 >= rows_a) break;
                            float gv = gate[e], uv = up[e];
                            if (bias != nullptr) {
                                gv += bias[i_row + e];
                                uv += bias[i_row + e + 8];
                            }
                            gv = round_as<TO>(gv);
                            uv = round_as<TO>(uv);
                            res[e] = silu_as<TO>(gv) * uv;
                            ++n_ok;
                        }
                        store4(out + (size_t)jj * ldo + (i_row >> 4) * 8 + (i_row & 7), res, n_ok);
                    }
                }
            } else {
                const int groups = share / 4;
                for (int idx = epi_tid; idx < groups * BN; idx += 128) {
                    const int col = idx / groups, row = row_begin + (idx % groups) * 4;   // rows fastest
                    const int i_row = a_row0 + row, jj = b_row0 + col;
                    if (i_row < rows_a && jj < rows_b) {
                        float v[4];
                        total4(row, col, v);
                        const int n_ok = rows_a - i_row < 4 ? rows_a - i_row : 4;
                        if (TRANSPOSED) {
                            if (bias != nullptr)
                                for (int e = 0; e < n_ok; ++e) v[e] += bias[i_row + e];
                            store4(out + (size_t)jj * ldo + i_row, v, n_ok);
                        } else {
                            const float bj = bias != nullptr ? bias[jj] : 0.f;
                            for (int e = 0; e < n_ok; ++e) out[(size_t)(i_row + e) * ldo + jj] = from_f<TO>(v[e] + bj);
                        }
                    }
                }
            }
        }
        cluster.sync();      // nobody's shared memory goes away while a peer still reads it
    }
    // ---- teardown: the tensor memory goes back whatever happened above ----
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d),
                     "r"((uint32_t)TMEM_COLS)
                     : "memory");
    }
}

template <int BN, bool TRANSPOSED, bool SWIGLU, typename TO>
cudaError_t launch_tc(dim3 grid, size_t smem, cudaStream_t stream, const CUtensorMap& ma,
                      const CUtensorMap& mb, TO* out, int64_t ldo, const float* bias, int rows_a,
                      int rows_b, int K, int stages, int splitk, int cluster_k) {
    auto kernel = gemm_tc_kernel<BN, TRANSPOSED, SWIGLU, TO>;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(TC_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int n = 0;
    if (tk_pdl_enabled()) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    if (cluster_k > 1) {
        attr[n].id = cudaLaunchAttributeClusterDimension;
        attr[n].val.clusterDim.x = 1;
        attr[n].val.clusterDim.y = 1;
        attr[n].val.clusterDim.z = cluster_k;
        ++n;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n;
    return cudaLaunchKernelEx(&cfg, kernel, ma, mb, out, ldo, bias, rows_a, rows_b, K, stages, splitk, cluster_k);
}

}  // namespace

// 0 if no tensor-core GEMM on the current device has given up on a barrier since the last call;
// else the place it gave up (1 producer, 2 MMA issuer, 3 epilogue). Resets the word.
TK_API int tk_gemm_tc_status() {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_tc_error, sizeof(int)) != cudaSuccess) return -1;
    if (v != 0) cudaMemcpyToSymbol(g_tc_error, &zero, sizeof(int));
    return v;
}

// Decode form: out[tokens, N] = x[tokens, K] . w[N, K]^T (+ bias[N]); tokens <= 256.
// swiglu: see gemm_skinny (rows of w in runs of 8 gate / 8 up; out is [tokens, N / 2]).
// split_k: whether K may be split over a cluster. out_dtype: bfloat16 or float.
TK_API int tk_gemm_tc_decode(const void* x, int64_t ldx, const void* w, int64_t ldw, const float* bias,
                             void* out, int64_t ldo, int tokens, int N, int K, int out_dtype, int swiglu,
                             int split_k, cudaStream_t stream) {
    TK_CHECK_ARG(tokens > 0 && tokens <= 256 && N > 0 && K > 0, "gemm_tc_decode: tokens=%d (1..256) N=%d K=%d",
                 tokens, N, K);
    TK_CHECK_ARG(K % 8 == 0 && ldx % 8 == 0 && ldw % 8 == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)w % 16 == 0,
                 "gemm_tc_decode: K and the leading dimensions must be multiples of 8, bases 16-byte aligned");
    TK_CHECK_ARG(!swiglu || N % 16 == 0, "gemm_tc_decode: the fused SwiGLU needs N (%d) in blocks of 16", N);
    const int BN = tokens <= 16 ? 16 : tokens <= 32 ? 32 : tokens <= 64 ? 64 : tokens <= 128 ? 128 : 256;
    CUtensorMap ma, mb;
    TK_CHECK_ARG(make_map(&ma, w, N, K, ldw, BM) && make_map(&mb, x, tokens, K, ldx, BN),
                 "gemm_tc_decode: cuTensorMapEncodeTiled failed (N=%d K=%d ldw=%lld)", N, K, (long long)ldw);
    const int a_tiles = (N + BM - 1) / BM;
    const int kb_total = (K + BK - 1) / BK;
    // split K until there are about two CTAs per SM's worth of slices (up to 16 tokens; one for
    // wider token tiles) or slices of 4 k-blocks, at most 8 ways: the partial tiles are reduced
    // inside a cluster. Measured on a B200 (2048- to 8192-wide matrices, CUDA graphs). The
    // pipeline takes at most ~100 KB so that two CTAs share an SM: one CTA's prologue and epilogue
    // hide behind the other's loads (head at 64 tokens: 64.8 us with one CTA per SM, 49.1 us
    // with two).
    constexpr int MIN_KB = 4, STAGE_KB = 100;
    int splitk = 1;
    const int target = BN <= 16 ? 2 * 148 : 148;
    while (split_k && splitk < 8 && a_tiles * splitk < target && kb_total / (splitk * 2) >= MIN_KB) splitk *= 2;
    const int cluster_k = splitk > 1 ? splitk : 0;
    const int kb_per = (kb_total + splitk - 1) / splitk;
    const int stage_bytes = A_TILE_BYTES + BN * BK * 2;
    int stages = kb_per < 6 ? kb_per : 6;
    while (stages > 2 && (size_t)stages * stage_bytes > (size_t)STAGE_KB * 1024) --stages;
    size_t smem = (size_t)stages * stage_bytes + (2 * stages + 2) * 8 + 1024 + 64;
    if (smem < (size_t)BN * BM * 4 + 1024 + 256) smem = (size_t)BN * BM * 4 + 1024 + 256;
    const dim3 grid(a_tiles, 1, splitk);
    cudaError_t err = cudaSuccess;
#define TK_TC(BN_, SW_, TO_)                                                                        \
    err = launch_tc<BN_, true, SW_, TO_>(grid, smem, stream, ma, mb, (TO_*)out, ldo, bias, N, tokens, K, \
                                         stages, splitk, cluster_k)
#define TK_TC_BN(SW_, TO_)                                                                          \
    switch (BN) {                                                                                   \
        case 16: TK_TC(16, SW_, TO_); break;                                                        \
        case 32: TK_TC(32, SW_, TO_); break;                                                        \
        case 64: TK_TC(64, SW_, TO_); break;                                                        \
        case 128: TK_TC(128, SW_, TO_); break;                                                      \
        default: TK_TC(256, SW_, TO_); break;                                                       \
    }
    if (out_dtype == TK_BF16) {
        if (swiglu) { TK_TC_BN(true, __nv_bfloat16) } else { TK_TC_BN(false, __nv_bfloat16) }
    } else if (out_dtype == TK_F32) {
        if (swiglu) { TK_TC_BN(true, float) } else { TK_TC_BN(false, float) }
    } else {
        TK_CHECK_ARG(false, "gemm_tc_decode: output dtype %d", out_dtype);
    }
#undef TK_TC_BN
#undef TK_TC
    if (err != cudaSuccess) {
        tk_set_error("gemm_tc_decode: launch failed: %s (tiles %d, splitk %d, stages %d, smem %zu)",
                     cudaGetErrorString(err), a_tiles, splitk, stages, smem);
        cudaGetLastError();
        return -2;
    }
    return 0;
}
