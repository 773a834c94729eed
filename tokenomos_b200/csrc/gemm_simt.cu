// C[M, N] = A[M, K] . W[N, K]^T (+ bias[N]) on the CUDA cores with 32-bit FMA accumulation.
// This is the matrix product of the true 32-bit path (no tensor cores, no reduced-precision
// mode can reach it), and the any-shape fallback of the 16-bit path (16-bit operands widen
// exactly, the sum stays 32-bit, the result is float or rounded once to 16-bit).
#include "common.cuh"

namespace {
constexpr int TM = 64, TN = 64, TK = 16, GEMM_THREADS = 256;
}

template <typename TA, typename TO>
__global__ void __launch_bounds__(GEMM_THREADS)
gemm_simt_kernel(const TA* A, int64_t lda, const TA* __restrict__ W, int64_t ldw,
                 const float* __restrict__ bias, TO* C, int64_t ldc, int M, int N,
                 int K) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float As[TK][TM + 4];
    __shared__ float Ws[TK][TN + 4];
    const int tid = threadIdx.x;
    const int m0 = blockIdx.y * TM, n0 = blockIdx.x * TN;
    const int tx = tid & 15, ty = tid >> 4;  // 16 x 16 threads, 4 x 4 outputs each
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    // each thread loads 4 elements of the A tile and 4 of the W tile: row = tid / 4, 4 k's
    const int lr = tid >> 2, lk = (tid & 3) * 4;
    for (int k0 = 0; k0 < K; k0 += TK) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int k = k0 + lk + e;
            const int m = m0 + lr, n = n0 + lr;
            As[lk + e][lr] = (m < M && k < K) ? to_f<TA>(A[(size_t)m * lda + k]) : 0.f;
            Ws[lk + e][lr] = (n < N && k < K) ? to_f<TA>(W[(size_t)n * ldw + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < TK; ++k) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[k][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = Ws[k][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + ty * 4 + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n >= N) continue;
            float v = acc[i][j];
            if (bias != nullptr) v += bias[n];
            C[(size_t)m * ldc + n] = from_f<TO>(v);
        }
    }
}

// in_dtype: operands A and W; out_dtype: C (float output from 16-bit operands is allowed,
// the head uses it). Leading dimensions in elements.
TK_API int tk_gemm_simt(const void* A, int64_t lda, const void* W, int64_t ldw, const float* bias,
                        void* C, int64_t ldc, int M, int N, int K, int in_dtype, int out_dtype,
                        cudaStream_t stream) {
    TK_CHECK_ARG(M >= 0 && N > 0 && K > 0, "gemm_simt: bad sizes M=%d N=%d K=%d", M, N, K);
    TK_CHECK_ARG(lda >= K && ldw >= K && ldc >= N, "gemm_simt: leading dimensions too small");
    if (M == 0) return 0;
    dim3 grid((N + TN - 1) / TN, (M + TM - 1) / TM);
    if (in_dtype == TK_F32 && out_dtype == TK_F32)
        tk_launch(gemm_simt_kernel<float, float>, dim3(grid), dim3(GEMM_THREADS), 0, stream, 
            (const float*)A, lda, (const float*)W, ldw, bias, (float*)C, ldc, M, N, K);
    else if (in_dtype == TK_BF16 && out_dtype == TK_BF16)
        tk_launch(gemm_simt_kernel<__nv_bfloat16, __nv_bfloat16>, dim3(grid), dim3(GEMM_THREADS), 0, stream, 
            (const __nv_bfloat16*)A, lda, (const __nv_bfloat16*)W, ldw, bias, (__nv_bfloat16*)C, ldc,
            M, N, K);
    else if (in_dtype == TK_BF16 && out_dtype == TK_F32)
        tk_launch(gemm_simt_kernel<__nv_bfloat16, float>, dim3(grid), dim3(GEMM_THREADS), 0, stream, 
            (const __nv_bfloat16*)A, lda, (const __nv_bfloat16*)W, ldw, bias, (float*)C, ldc, M, N, K);
    else
        TK_CHECK_ARG(false, "gemm_simt: dtype pair (%d, %d) is not built", in_dtype, out_dtype);
    TK_CHECK_LAUNCH("gemm_simt");
    return 0;
}
