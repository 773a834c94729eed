// Skinny matrix product for decoding: out[M, N] = x[M, K] . W[N, K]^T (+ bias) with M <= 16
// tokens, bfloat16 operands, 32-bit accumulation on the tensor cores (mma.sync m16n8k16 with the
// weight rows on the M axis: the few tokens are the N axis, so no tensor-core lane is wasted on
// padding the batch to 128 rows).
//
// Such a product is a stream of weight bytes and nothing else, so the kernel is built around
// loads: a CTA owns 16 weight rows and all of K; its warps take alternate 64-wide slices of K;
// every thread reads its share of the weight rows with 16-byte loads straight into registers
// (each row is read as whole 128-byte lines), all slices of a warp in flight at once, and the
// same 16-byte pattern of the activations, which stay in L1/L2. The K index a register pair
// stands for is permuted, identically for both operands, so that one 16-byte load feeds two
// mma steps without any shuffle. Warps then add their partial sums through shared memory.
#include "common.cuh"

namespace {

__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                         uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
        "{%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 ldg_stream(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

// Activations are written by the kernel before this one, which may still be running when this
// kernel's blocks become resident: they must not go through the read-only (.nc) path, whose
// lines are not refreshed by griddepcontrol.wait.
__device__ __forceinline__ uint4 ld_activation(const void* p) {
    uint4 v;
    asm volatile("ld.global.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p)
                 : "memory");
    return v;
}

constexpr int ROWS = 16;     // weight rows per CTA
constexpr int KSLICE = 64;   // K elements a warp takes per iteration (128 bytes of each row)

// What the short-conv epilogue needs beside the product (EPI_CONV): the depthwise taps, the
// per-request state rows and where each token's request keeps them.
struct ConvTail {
    const float* taps;        // [d, W]
    const float* bias;        // [d] or null
    __nv_bfloat16* state;     // [slots, W - 1, d]
    const int* seq_ctx;       // [M] tokens already cached (0: the state row reads as zeros)
    const int* seq_slot;      // [M]
    int W, d;
};

enum : int { EPI_NONE = 0, EPI_SWIGLU = 1, EPI_CONV = 2 };

// The two halves of a residual add + RMSNorm taken into the products on either side of it, so
// that a decode step needs no kernel between two products:
//   NORM (the product after the norm): x is the residual stream itself, not normed. Every CTA
//     reads all of x anyway, so it sums the squares of what it loads, and the epilogue scales the
//     accumulators by rstd = 1 / sqrt(mean(x^2) + eps) of each token's row. The norm's weight is
//     folded into the matrix's columns when the model is built (W'[n, k] = W[n, k] * weight[k]),
//     so (x * rstd * weight) . W^T = rstd * (x . W'^T).
//   ADD (the product before the norm): the epilogue adds the product, rounded as a store would
//     round it, to `residual` and writes the new stream, rounded once: what the norm kernel's
//     add does.
struct Fuse {
    float eps;                          // NORM
    const __nv_bfloat16* residual;      // ADD: [M, N], rows `ldr` apart
    int64_t ldr;
};

__device__ __forceinline__ float sum_squares(const uint4& v) {
    float acc = 0.f;
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[i]));
        acc = fmaf(f.x, f.x, acc);
        acc = fmaf(f.y, f.y, acc);
    }
    return acc;
}

// MT: 8 or 16 tokens (one or two n8 tiles). R8: the CTA owns 8 weight rows instead of 16 (the
// upper half of the mma tile stays zero): twice as many CTAs for matrices with few rows.
// EPI_SWIGLU: the weight rows come in blocks of 16, 8 gate rows then the 8 up rows of the same
// channels, and the CTA writes silu(gate) * up for its 8 channels: out is [M, N / 2].
// EPI_CONV: the weight rows come in blocks of 24 (8 rows of B, of C and of X of the same 8
// channels of a gated short conv), every token is a sequence of its own with one new token, and
// the CTA writes C * conv(B * X) for its 8 channels and moves their state on: out is [M, N / 3].
// A second mma per step takes the X rows (its upper half stays zero).
// UNROLL: slices whose loads a warp has in flight together (registers: 8 per slice and row half)
template <int MT, typename TO, bool R8, int EPI, int UNROLL, bool NORM = false, bool ADD = false>
__global__ void __launch_bounds__(512)
gemm_skinny_kernel(const __nv_bfloat16* x, int64_t ldx,
                   const __nv_bfloat16* __restrict__ w, int64_t ldw, const float* __restrict__ bias,
                   TO* out, int64_t ldo, int M, int N, int K, ConvTail tail, Fuse fuse) {
    extern __shared__ float red[];                 // [warps][RED_ROWS][MT], NORM: + [warps][MT] + [MT]
    pdl_launch_dependents();
    constexpr bool SWIGLU = EPI == EPI_SWIGLU, CONV = EPI == EPI_CONV;
    constexpr int RED_ROWS = CONV ? 24 : ROWS;
    const int warps = blockDim.x >> 5;
    float* ssq_s = red + (size_t)warps * RED_ROWS * MT;      // NORM: each warp's sums of squares
    float* rstd_s = ssq_s + (size_t)warps * MT;              // NORM: 1 / rms of each token's row
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    constexpr int CTA_ROWS = CONV ? 24 : (R8 ? 8 : ROWS);
    const int n0 = blockIdx.x * CTA_ROWS;
    const int r0 = n0 + g, r1 = n0 + g + 8, r2 = n0 + g + 16;
    const bool r0_ok = r0 < N, r1_ok = !R8 && r1 < N, r2_ok = CONV && r2 < N;
    const __nv_bfloat16* w0 = w + (size_t)(r0_ok ? r0 : 0) * ldw;
    const __nv_bfloat16* w1 = w + (size_t)(r1_ok ? r1 : 0) * ldw;
    const __nv_bfloat16* w2 = w + (size_t)(r2_ok ? r2 : 0) * ldw;
    constexpr int TG = MT / 8;
    const __nv_bfloat16* xr[TG];
    bool x_ok[TG];
#pragma unroll
    for (int i = 0; i < TG; ++i) {
        const int tok = 8 * i + g;
        x_ok[i] = tok < M;
        xr[i] = x + (size_t)(x_ok[i] ? tok : 0) * ldx;
    }
    float acc[TG][4], accx[CONV ? TG : 1][4];
#pragma unroll
    for (int i = 0; i < TG; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[i][e] = 0.f;
#pragma unroll
    for (int i = 0; i < (CONV ? TG : 1); ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) accx[i][e] = 0.f;

    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
    const int slices = (K + KSLICE - 1) / KSLICE;
    bool waited = false;
    float pf_state[3] = {0.f, 0.f, 0.f};
    int pf_ctx = 0;
    bool pf = false;
    float ss[TG];                                  // NORM: this thread's share of sum(x^2)
#pragma unroll
    for (int i = 0; i < TG; ++i) ss[i] = 0.f;
    float pf_res = 0.f;                            // ADD: the residual of this thread's output
    bool pf_res_ok = false;
    for (int s0 = warp; s0 < slices; s0 += warps * UNROLL) {
        uint4 wa[UNROLL][2], wb[UNROLL][2], wc[CONV ? UNROLL : 1][2];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int s = s0 + u * warps;
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int k = s * KSLICE + h * 32 + 8 * t;
                const bool ok = s < slices && k < K;
                wa[u][h] = (ok && r0_ok) ? ldg_stream(w0 + k) : zero;
                wb[u][h] = (ok && r1_ok) ? ldg_stream(w1 + k) : zero;
                if constexpr (CONV) wc[u][h] = (ok && r2_ok) ? ldg_stream(w2 + k) : zero;
            }
        }
        // the weights do not depend on the kernel before this one: their loads are in flight
        // while it finishes; the activations do, so wait before the first of them
        if (!waited) {
            pdl_wait();
            waited = true;
            if constexpr (ADD) {
                // the residual this thread's output joins, asked for now instead of after the
                // reduction (rows fastest, as the epilogue walks them)
                constexpr int CR = R8 ? 8 : ROWS;
                const int tok = threadIdx.x / CR, r = threadIdx.x % CR;
                if ((int)threadIdx.x < CR * MT && tok < M && n0 + r < N) {
                    pf_res = __bfloat162float(fuse.residual[(size_t)tok * fuse.ldr + n0 + r]);
                    pf_res_ok = true;
                }
            }
            if constexpr (CONV) {
                // what this thread's (token, channel) needs of the conv state in the epilogue is
                // asked for now (widths up to 4): two trips to memory, one behind the other, that
                // would otherwise follow the reduction at the kernel's tail
                const int tok = threadIdx.x / 8, c = blockIdx.x * 8 + threadIdx.x % 8;
                if (threadIdx.x < 8 * MT && tok < M && c < tail.d && tail.W <= 4) {
                    pf_ctx = tail.seq_ctx[tok];
                    const __nv_bfloat16* st = tail.state + (size_t)TK_SLOT(TK_K_SKINNY_CONV, tail.seq_slot[tok]) * (tail.W - 1) * tail.d + c;
#pragma unroll
                    for (int k = 0; k < 3; ++k)
                        if (k < tail.W - 1) pf_state[k] = __bfloat162float(st[(size_t)k * tail.d]);
                    pf = true;
                }
            }
        }
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int s = s0 + u * warps;
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int k = s * KSLICE + h * 32 + 8 * t;
                const bool ok = s < slices && k < K;
#pragma unroll
                for (int i = 0; i < TG; ++i) {
                    const uint4 xv = (ok && x_ok[i]) ? ld_activation(xr[i] + k) : zero;
                    if constexpr (NORM) ss[i] += sum_squares(xv);
                    // elements 0..3 of the 16 bytes are one mma step, 4..7 the next
                    mma16816(acc[i], wa[u][h].x, wb[u][h].x, wa[u][h].y, wb[u][h].y, xv.x, xv.y);
                    mma16816(acc[i], wa[u][h].z, wb[u][h].z, wa[u][h].w, wb[u][h].w, xv.z, xv.w);
                    if constexpr (CONV) {
                        mma16816(accx[i], wc[u][h].x, 0u, wc[u][h].y, 0u, xv.x, xv.y);
                        mma16816(accx[i], wc[u][h].z, 0u, wc[u][h].w, 0u, xv.z, xv.w);
                    }
                }
            }
        }
    }
    if (!waited) pdl_wait();
    // acc[i]: rows g / g + 8, tokens 8 i + 2 t, + 1
#pragma unroll
    for (int i = 0; i < TG; ++i) {
        float* dst = red + (size_t)warp * RED_ROWS * MT;
        dst[g * MT + 8 * i + 2 * t] = acc[i][0];
        dst[g * MT + 8 * i + 2 * t + 1] = acc[i][1];
        dst[(g + 8) * MT + 8 * i + 2 * t] = acc[i][2];
        dst[(g + 8) * MT + 8 * i + 2 * t + 1] = acc[i][3];
        if constexpr (CONV) {
            dst[(g + 16) * MT + 8 * i + 2 * t] = accx[i][0];
            dst[(g + 16) * MT + 8 * i + 2 * t + 1] = accx[i][1];
        }
    }
    if constexpr (NORM) {
        // lanes t = 0..3 of a quad hold parts of token g's sum; the CTA's warps cover all of K
#pragma unroll
        for (int i = 0; i < TG; ++i) {
            float v = ss[i];
            v += __shfl_xor_sync(0xffffffffu, v, 1);
            v += __shfl_xor_sync(0xffffffffu, v, 2);
            if (t == 0) ssq_s[warp * MT + 8 * i + g] = v;
        }
    }
    __syncthreads();
    if constexpr (NORM) {
        if ((int)threadIdx.x < MT) {
            float v = 0.f;
            for (int wv = 0; wv < warps; ++wv) v += ssq_s[wv * MT + threadIdx.x];
            rstd_s[threadIdx.x] = rsqrtf(v / (float)K + fuse.eps);
        }
        __syncthreads();
    }
    if constexpr (CONV) {
        // one thread per (token, channel): B, C, X of the channel as the unfused path stores them,
        // u = B X, the taps over the state row and u, the state moved on by one
        const int W = tail.W, d = tail.d;
        for (int idx = threadIdx.x; idx < 8 * MT; idx += blockDim.x) {
            const int tok = idx / 8, j = idx % 8;
            const int c = blockIdx.x * 8 + j;
            if (tok >= M || c >= d) continue;
            float bv = 0.f, cv = 0.f, xv = 0.f;
            for (int wv = 0; wv < warps; ++wv) {
                const float* src = red + (size_t)wv * RED_ROWS * MT + tok;
                bv += src[j * MT];
                cv += src[(j + 8) * MT];
                xv += src[(j + 16) * MT];
            }
            if constexpr (NORM) {
                const float rs = rstd_s[tok];
                bv *= rs;
                cv *= rs;
                xv *= rs;
            }
            if (bias != nullptr) {
                bv += bias[n0 + j];
                cv += bias[n0 + 8 + j];
                xv += bias[n0 + 16 + j];
            }
            bv = round_as<TO>(bv);
            cv = round_as<TO>(cv);
            xv = round_as<TO>(xv);
            const float u = round_as<TO>(bv * xv);
            const bool have = pf && idx == (int)threadIdx.x;          // fetched at the start
            const int ctx = have ? pf_ctx : tail.seq_ctx[tok];
            __nv_bfloat16* st = tail.state + (size_t)TK_SLOT(TK_K_SKINNY_CONV, tail.seq_slot[tok]) * (W - 1) * d + c;
            const float* taps = tail.taps + (size_t)c * W;
            // state row k holds u of position ctx - (W - 1) + k; before position 0 it reads as 0
            float acc_c = 0.f;
            if (have) {
#pragma unroll
                for (int k = 0; k < 3; ++k) {
                    if (k < W - 1) {
                        const float hv = ctx - (W - 1) + k < 0 ? 0.f : pf_state[k];
                        acc_c += hv * taps[k];
                        if (k > 0) st[(size_t)(k - 1) * d] = __float2bfloat16_rn(hv);
                    }
                }
            } else {
                for (int k = 0; k < W - 1; ++k) {
                    const float hv = ctx - (W - 1) + k < 0 ? 0.f : __bfloat162float(st[(size_t)k * d]);
                    acc_c += hv * taps[k];
                    // row k - 1 takes what row k held (it was read in the pass before this one)
                    if (k > 0) st[(size_t)(k - 1) * d] = __float2bfloat16_rn(hv);
                }
            }
            st[(size_t)(W - 2) * d] = __float2bfloat16_rn(u);
            acc_c += u * taps[W - 1];
            if (tail.bias != nullptr) acc_c += tail.bias[c];
            const float y = round_as<TO>(acc_c);
            out[(size_t)tok * ldo + c] = from_f<TO>(cv * y);
        }
    } else if constexpr (SWIGLU) {
        for (int idx = threadIdx.x; idx < 8 * MT; idx += blockDim.x) {
            const int tok = idx / 8, j = idx % 8;
            if (tok >= M || n0 + 8 + j >= N) continue;
            float gate = 0.f, up = 0.f;
            for (int wv = 0; wv < warps; ++wv) {
                gate += red[(size_t)wv * ROWS * MT + j * MT + tok];
                up += red[(size_t)wv * ROWS * MT + (j + 8) * MT + tok];
            }
            if constexpr (NORM) {
                gate *= rstd_s[tok];
                up *= rstd_s[tok];
            }
            if (bias != nullptr) {
                gate += bias[n0 + j];
                up += bias[n0 + 8 + j];
            }
            // the unfused path stores gate and up in the output type, then rounds silu(gate)
            gate = round_as<TO>(gate);
            up = round_as<TO>(up);
            const float act = silu_as<TO>(gate);
            out[(size_t)tok * ldo + n0 / 2 + j] = from_f<TO>(act * up);
        }
    } else {
        for (int idx = threadIdx.x; idx < CTA_ROWS * MT; idx += blockDim.x) {
            const int tok = idx / CTA_ROWS, r = idx % CTA_ROWS;   // rows fastest: neighbours in memory
            if (tok >= M || n0 + r >= N) continue;
            float v = 0.f;
            for (int wv = 0; wv < warps; ++wv) v += red[(size_t)wv * ROWS * MT + r * MT + tok];
            if constexpr (NORM) v *= rstd_s[tok];
            if (bias != nullptr) v += bias[n0 + r];
            if constexpr (ADD) {
                const float res = (pf_res_ok && idx == (int)threadIdx.x)
                                      ? pf_res
                                      : __bfloat162float(fuse.residual[(size_t)tok * fuse.ldr + n0 + r]);
                v = res + round_as<TO>(v);
            }
            out[(size_t)tok * ldo + n0 + r] = from_f<TO>(v);
        }
    }
}

}  // namespace

// How the launch is shaped, measured on a B200 in CUDA graphs at 1 and 8 tokens (2048- and
// 8192-wide K): two slices in flight per warp beat four (75 instead of 126 registers: three CTAs
// of 8 warps per SM instead of two, whose load, compute and reduce phases overlap); a tall matrix
// (300 or more CTAs) wants 8 warps per CTA, a short one 16 (more of K in flight per CTA); 8-row
// CTAs only pay below half a wave.
// x: [M, K] bfloat16, rows `ldx` apart; w: [N, K] bfloat16, rows `ldw` apart; out: [M, N]
// bfloat16 or float (out_dtype); M <= 16; K, ldx, ldw multiples of 8 and 16-byte aligned bases.
// swiglu != 0: w holds blocks of 8 gate rows followed by the 8 up rows of the same channels
// (N a multiple of 16) and out is [M, N / 2] = silu(gate) * up.
// norm_eps > 0 (at most 8 rows, bfloat16 out): x is an un-normed stream and the result is scaled
// by each row's 1 / sqrt(mean(x^2) + norm_eps) (see Fuse; the norm's weight is in w's columns).
// residual != null (at most 8 rows, bfloat16 out, no swiglu): out = residual + product, the
// product rounded first, the sum rounded once; residual: [M, N] bfloat16, rows `ldr` apart.
TK_API int tk_gemm_skinny(const void* x, int64_t ldx, const void* w, int64_t ldw, const float* bias,
                          void* out, int64_t ldo, int M, int N, int K, int out_dtype, int swiglu,
                          float norm_eps, const void* residual, int64_t ldr, cudaStream_t stream) {
    TK_CHECK_ARG(M >= 0 && M <= 16 && N > 0 && K > 0, "gemm_skinny: M=%d (at most 16) N=%d K=%d", M, N, K);
    TK_CHECK_ARG(K % 8 == 0 && ldx % 8 == 0 && ldw % 8 == 0, "gemm_skinny: K and the leading dimensions "
                 "must be multiples of 8 (K=%d)", K);
    TK_CHECK_ARG(((uintptr_t)x % 16 == 0) && ((uintptr_t)w % 16 == 0), "gemm_skinny: operands must be 16-byte aligned");
    TK_CHECK_ARG(!swiglu || N % 16 == 0, "gemm_skinny: the fused SwiGLU needs N (%d) in blocks of 16", N);
    const bool norm = norm_eps > 0.f, add = residual != nullptr;
    TK_CHECK_ARG(!(norm || add) || (M <= 8 && out_dtype == TK_BF16),
                 "gemm_skinny: the fused norm and the fused residual add take at most 8 rows and a "
                 "bfloat16 output (M=%d)", M);
    TK_CHECK_ARG(!(norm && add) && !(add && swiglu), "gemm_skinny: the residual add goes with a plain product only");
    if (M == 0) return 0;
    const int slices = (K + KSLICE - 1) / KSLICE;
    const int ctas16 = (N + ROWS - 1) / ROWS;
    // between one and two waves of 16-row CTAs, and a short K: 8-row CTAs with four slices in
    // flight (the 3072 x 2048 qkv projection: 3.5 us against 4.9)
    const bool mid = !swiglu && ctas16 >= 160 && ctas16 < 296 && K <= 4096;
    const int unroll = mid ? 4 : 2;
    const int max_warps = ctas16 >= 296 || mid ? 8 : 16;
    int warps = (slices + unroll - 1) / unroll;      // every slice of a warp in flight at once
    warps = warps < 1 ? 1 : (warps > max_warps ? max_warps : warps);
    const int threads = warps * 32;
    // very few rows: 8 per CTA so that the grid still covers the GPU
    const bool r8 = !swiglu && (mid || ctas16 < 74);
    const int blocks = r8 ? (N + 7) / 8 : (N + ROWS - 1) / ROWS;
    const int MT = M <= 8 ? 8 : 16;
    const size_t smem = ((size_t)warps * ROWS * MT + (norm ? (size_t)warps * MT + MT : 0)) * sizeof(float);
    auto x_ = (const __nv_bfloat16*)x;
    auto w_ = (const __nv_bfloat16*)w;
    const Fuse fuse{norm_eps, (const __nv_bfloat16*)residual, ldr};
#define TK_SKINNY_F(MT_, TO_, R8_, SW_, NORM_, ADD_)                                               \
    do {                                                                                           \
        if (unroll == 2)                                                                           \
            tk_launch(gemm_skinny_kernel<MT_, TO_, R8_, SW_, 2, NORM_, ADD_>, dim3(blocks), dim3(threads), smem, \
                      stream, x_, ldx, w_, ldw, bias, (TO_*)out, ldo, M, N, K, ConvTail{}, fuse);   \
        else                                                                                       \
            tk_launch(gemm_skinny_kernel<MT_, TO_, R8_, SW_, 4, NORM_, ADD_>, dim3(blocks), dim3(threads), smem, \
                      stream, x_, ldx, w_, ldw, bias, (TO_*)out, ldo, M, N, K, ConvTail{}, fuse);   \
    } while (0)
#define TK_SKINNY(MT_, TO_, R8_, SW_) TK_SKINNY_F(MT_, TO_, R8_, SW_, false, false)
#define TK_SKINNY_T(TO_)                                                                           \
    do {                                                                                           \
        if (swiglu) { if (MT == 8) TK_SKINNY(8, TO_, false, EPI_SWIGLU); else TK_SKINNY(16, TO_, false, EPI_SWIGLU); } \
        else if (r8) { if (MT == 8) TK_SKINNY(8, TO_, true, EPI_NONE); else TK_SKINNY(16, TO_, true, EPI_NONE); } \
        else { if (MT == 8) TK_SKINNY(8, TO_, false, EPI_NONE); else TK_SKINNY(16, TO_, false, EPI_NONE); }  \
    } while (0)
    if (norm) {
        if (swiglu) TK_SKINNY_F(8, __nv_bfloat16, false, EPI_SWIGLU, true, false);
        else if (r8) TK_SKINNY_F(8, __nv_bfloat16, true, EPI_NONE, true, false);
        else TK_SKINNY_F(8, __nv_bfloat16, false, EPI_NONE, true, false);
    } else if (add) {
        if (r8) TK_SKINNY_F(8, __nv_bfloat16, true, EPI_NONE, false, true);
        else TK_SKINNY_F(8, __nv_bfloat16, false, EPI_NONE, false, true);
    } else if (out_dtype == TK_BF16) TK_SKINNY_T(__nv_bfloat16);
    else if (out_dtype == TK_F32) TK_SKINNY_T(float);
    else TK_CHECK_ARG(false, "gemm_skinny: output dtype %d", out_dtype);
#undef TK_SKINNY_T
#undef TK_SKINNY
#undef TK_SKINNY_F
    TK_CHECK_LAUNCH("gemm_skinny");
    return 0;
}

// The in-projection of a gated short conv with the conv in its epilogue, for a step in which every
// token is a sequence of its own with one new token (decoding). x: [M, K] bfloat16, M <= 16;
// w: [3 d, K] bfloat16 whose rows come in blocks of 24: 8 rows of B, of C and of X of the same 8
// channels (d a multiple of 8); bias: [3 d] in the same order, or null. taps: [d, W] float32,
// conv_bias: [d] or null; state: [slots, W - 1, d] bfloat16, moved on by one token per request;
// seq_ctx, seq_slot: [M]. out: [M, d] bfloat16 = C * conv(B * X). norm_eps > 0: x is an un-normed
// stream and B, C, X are scaled by each row's 1 / rms first (see tk_gemm_skinny).
TK_API int tk_gemm_skinny_conv(const void* x, int64_t ldx, const void* w, int64_t ldw, const float* bias,
                               void* out, int64_t ldo, int M, int d, int K, const float* taps,
                               const float* conv_bias, void* state, const int* seq_ctx,
                               const int* seq_slot, int W, float norm_eps, cudaStream_t stream) {
    TK_CHECK_ARG(M >= 0 && M <= 16 && d > 0 && K > 0, "gemm_skinny_conv: M=%d (at most 16) d=%d K=%d", M, d, K);
    TK_CHECK_ARG(K % 8 == 0 && ldx % 8 == 0 && ldw % 8 == 0, "gemm_skinny_conv: K and the leading "
                 "dimensions must be multiples of 8 (K=%d)", K);
    TK_CHECK_ARG(((uintptr_t)x % 16 == 0) && ((uintptr_t)w % 16 == 0), "gemm_skinny_conv: operands must be 16-byte aligned");
    TK_CHECK_ARG(d % 8 == 0, "gemm_skinny_conv: the channel count (%d) must come in blocks of 8", d);
    TK_CHECK_ARG(W >= 2 && W <= 8, "gemm_skinny_conv: width %d outside 2..8", W);
    const bool norm = norm_eps > 0.f;
    TK_CHECK_ARG(!norm || M <= 8, "gemm_skinny_conv: the fused norm takes at most 8 rows (M=%d)", M);
    if (M == 0) return 0;
    const int N = 3 * d;
    const int slices = (K + KSLICE - 1) / KSLICE;
    const int blocks = d / 8;
    const int unroll = 2;
    // (90 registers: two CTAs of 8 warps per SM. Bounding it to 80 for three made the decode step
    // slower, 0.842 ms against 0.816 ms.)
    const int max_warps = blocks >= 200 ? 8 : 16;
    int warps = (slices + unroll - 1) / unroll;
    warps = warps < 1 ? 1 : (warps > max_warps ? max_warps : warps);
    const int MT = M <= 8 ? 8 : 16;
    const size_t smem = ((size_t)warps * 24 * MT + (norm ? (size_t)warps * MT + MT : 0)) * sizeof(float);
    const ConvTail tail{taps, conv_bias, (__nv_bfloat16*)state, seq_ctx, seq_slot, W, d};
    const Fuse fuse{norm_eps, nullptr, 0};
    auto x_ = (const __nv_bfloat16*)x;
    auto w_ = (const __nv_bfloat16*)w;
    auto o_ = (__nv_bfloat16*)out;
#define TK_SKINNY_CONV(MT_, U_, NORM_)                                                             \
    tk_launch(gemm_skinny_kernel<MT_, __nv_bfloat16, false, EPI_CONV, U_, NORM_, false>, dim3(blocks),    \
              dim3(warps * 32), smem, stream, x_, ldx, w_, ldw, bias, o_, ldo, M, N, K, tail, fuse)
    if (norm) TK_SKINNY_CONV(8, 2, true);
    else if (MT == 8) TK_SKINNY_CONV(8, 2, false);
    else TK_SKINNY_CONV(16, 2, false);
#undef TK_SKINNY_CONV
    TK_CHECK_LAUNCH("gemm_skinny_conv");
    return 0;
}
