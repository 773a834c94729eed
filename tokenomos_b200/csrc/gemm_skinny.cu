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

__device__ __forceinline__ uint4 ldg_cached(const void* p) {
    return __ldg(reinterpret_cast<const uint4*>(p));
}

constexpr int ROWS = 16;     // weight rows per CTA
constexpr int KSLICE = 64;   // K elements a warp takes per iteration (128 bytes of each row)
constexpr int UNROLL = 4;    // slices whose loads are in flight together

// MT: 8 or 16 tokens (one or two n8 tiles)
template <int MT, typename TO>
__global__ void __launch_bounds__(512)
gemm_skinny_kernel(const __nv_bfloat16* __restrict__ x, int64_t ldx,
                   const __nv_bfloat16* __restrict__ w, int64_t ldw, const float* __restrict__ bias,
                   TO* __restrict__ out, int64_t ldo, int M, int N, int K) {
    extern __shared__ float red[];                 // [warps][ROWS][MT]
    const int warps = blockDim.x >> 5;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int n0 = blockIdx.x * ROWS;
    const int r0 = n0 + g, r1 = n0 + g + 8;
    const bool r0_ok = r0 < N, r1_ok = r1 < N;
    const __nv_bfloat16* w0 = w + (size_t)(r0_ok ? r0 : 0) * ldw;
    const __nv_bfloat16* w1 = w + (size_t)(r1_ok ? r1 : 0) * ldw;
    constexpr int TG = MT / 8;
    const __nv_bfloat16* xr[TG];
    bool x_ok[TG];
#pragma unroll
    for (int i = 0; i < TG; ++i) {
        const int tok = 8 * i + g;
        x_ok[i] = tok < M;
        xr[i] = x + (size_t)(x_ok[i] ? tok : 0) * ldx;
    }
    float acc[TG][4];
#pragma unroll
    for (int i = 0; i < TG; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[i][e] = 0.f;

    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
    const int slices = (K + KSLICE - 1) / KSLICE;
    for (int s0 = warp; s0 < slices; s0 += warps * UNROLL) {
        uint4 wa[UNROLL][2], wb[UNROLL][2];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int s = s0 + u * warps;
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int k = s * KSLICE + h * 32 + 8 * t;
                const bool ok = s < slices && k < K;
                wa[u][h] = (ok && r0_ok) ? ldg_stream(w0 + k) : zero;
                wb[u][h] = (ok && r1_ok) ? ldg_stream(w1 + k) : zero;
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
                    const uint4 xv = (ok && x_ok[i]) ? ldg_cached(xr[i] + k) : zero;
                    // elements 0..3 of the 16 bytes are one mma step, 4..7 the next
                    mma16816(acc[i], wa[u][h].x, wb[u][h].x, wa[u][h].y, wb[u][h].y, xv.x, xv.y);
                    mma16816(acc[i], wa[u][h].z, wb[u][h].z, wa[u][h].w, wb[u][h].w, xv.z, xv.w);
                }
            }
        }
    }
    // acc[i]: rows g / g + 8, tokens 8 i + 2 t, + 1
#pragma unroll
    for (int i = 0; i < TG; ++i) {
        float* dst = red + (size_t)warp * ROWS * MT;
        dst[g * MT + 8 * i + 2 * t] = acc[i][0];
        dst[g * MT + 8 * i + 2 * t + 1] = acc[i][1];
        dst[(g + 8) * MT + 8 * i + 2 * t] = acc[i][2];
        dst[(g + 8) * MT + 8 * i + 2 * t + 1] = acc[i][3];
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < ROWS * MT; idx += blockDim.x) {
        const int tok = idx / ROWS, r = idx % ROWS;      // rows fastest: neighbours in memory
        if (tok >= M || n0 + r >= N) continue;
        float v = 0.f;
        for (int wv = 0; wv < warps; ++wv) v += red[(size_t)wv * ROWS * MT + r * MT + tok];
        if (bias != nullptr) v += bias[n0 + r];
        out[(size_t)tok * ldo + n0 + r] = from_f<TO>(v);
    }
}

}  // namespace

// x: [M, K] bfloat16, rows `ldx` apart; w: [N, K] bfloat16, rows `ldw` apart; out: [M, N]
// bfloat16 or float (out_dtype); M <= 16; K, ldx, ldw multiples of 8 and 16-byte aligned bases.
TK_API int tk_gemm_skinny(const void* x, int64_t ldx, const void* w, int64_t ldw, const float* bias,
                          void* out, int64_t ldo, int M, int N, int K, int out_dtype,
                          cudaStream_t stream) {
    TK_CHECK_ARG(M >= 0 && M <= 16 && N > 0 && K > 0, "gemm_skinny: M=%d (at most 16) N=%d K=%d", M, N, K);
    TK_CHECK_ARG(K % 8 == 0 && ldx % 8 == 0 && ldw % 8 == 0, "gemm_skinny: K and the leading dimensions "
                 "must be multiples of 8 (K=%d)", K);
    TK_CHECK_ARG(((uintptr_t)x % 16 == 0) && ((uintptr_t)w % 16 == 0), "gemm_skinny: operands must be 16-byte aligned");
    if (M == 0) return 0;
    const int slices = (K + KSLICE - 1) / KSLICE;
    int warps = (slices + UNROLL - 1) / UNROLL;      // every slice of a warp in flight at once
    warps = warps < 1 ? 1 : (warps > 16 ? 16 : warps);
    const int threads = warps * 32;
    const int blocks = (N + ROWS - 1) / ROWS;
    const int MT = M <= 8 ? 8 : 16;
    const size_t smem = (size_t)warps * ROWS * MT * sizeof(float);
    auto x_ = (const __nv_bfloat16*)x;
    auto w_ = (const __nv_bfloat16*)w;
#define TK_SKINNY(MT_, TO_)                                                                         \
    gemm_skinny_kernel<MT_, TO_><<<blocks, threads, smem, stream>>>(x_, ldx, w_, ldw, bias, (TO_*)out, ldo, M, N, K)
    if (out_dtype == TK_BF16) {
        if (MT == 8) TK_SKINNY(8, __nv_bfloat16); else TK_SKINNY(16, __nv_bfloat16);
    } else if (out_dtype == TK_F32) {
        if (MT == 8) TK_SKINNY(8, float); else TK_SKINNY(16, float);
    } else {
        TK_CHECK_ARG(false, "gemm_skinny: output dtype %d", out_dtype);
    }
#undef TK_SKINNY
    TK_CHECK_LAUNCH("gemm_skinny");
    return 0;
}
