// Row-wise kernels of the residual stream: embedding / row gather, residual add + RMSNorm,
// SwiGLU, and the per-head sigmoid gate. Storage is float or bfloat16; statistics, sums and
// products are formed in 32-bit and rounded where the 16-bit reference rounds
// (Tokenomos kernels/norm/fused.py:22-28,69-82; models/blocks/ffn.py:31).
#include "common.cuh"

// ---------------------------------------------------------------------------------------------
// gather: out[r, :] = table[ids[r], :]  (embedding lookup, and row selection before the head)
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void gather_rows_kernel(const T* table, const int* ids,
                                   T* out, int width, int rows_in_table) {
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x;
    int id = TK_ROW(TK_K_GATHER, ids[r], rows_in_table);
    // an id outside the table would read foreign memory: clamp (callers validate on the host)
    id = id < 0 ? 0 : (id >= rows_in_table ? rows_in_table - 1 : id);
    const T* src = table + (size_t)id * width;
    T* dst = out + (size_t)r * width;
    constexpr int VEC = 16 / sizeof(T);
    if (width % VEC == 0) {
        const uint4* s4 = reinterpret_cast<const uint4*>(src);
        uint4* d4 = reinterpret_cast<uint4*>(dst);
        for (int i = threadIdx.x; i < width / VEC; i += blockDim.x) d4[i] = s4[i];
    } else {
        for (int i = threadIdx.x; i < width; i += blockDim.x) dst[i] = src[i];
    }
}

TK_API int tk_gather_rows(const void* table, const int* ids, void* out, int rows, int width,
                          int rows_in_table, int dtype, cudaStream_t stream) {
    TK_CHECK_ARG(rows >= 0 && width > 0 && rows_in_table > 0, "gather_rows: bad sizes rows=%d width=%d table=%d",
                 rows, width, rows_in_table);
    if (rows == 0) return 0;
    const int threads = width >= 1024 ? 256 : 128;
    if (dtype == TK_F32)
        tk_launch(gather_rows_kernel<float>, dim3(rows), dim3(threads), 0, stream, (const float*)table, ids, (float*)out,
                                                               width, rows_in_table);
    else if (dtype == TK_BF16)
        tk_launch(gather_rows_kernel<__nv_bfloat16>, dim3(rows), dim3(threads), 0, stream, 
            (const __nv_bfloat16*)table, ids, (__nv_bfloat16*)out, width, rows_in_table);
    else
        TK_CHECK_ARG(false, "gather_rows: unknown dtype %d", dtype);
    TK_CHECK_LAUNCH("gather_rows");
    return 0;
}

// The decode step's embedding lookup with the choice of the id in the same kernel: row r reads
// the token the step before sampled for its sequence (last_token[slot[r]]) when use_prev[r] is
// set, else the id the host gave; so a step can be queued before the host has seen that token.
template <typename T>
__global__ void gather_rows_select_kernel(const T* table, const int* ids_host, const int* use_prev,
                                          const int* last_token, const int* slot, T* out, int width,
                                          int rows_in_table) {
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x;
    int id = TK_ROW(TK_K_GATHER, use_prev[r] ? last_token[slot[r]] : ids_host[r], rows_in_table);
    id = id < 0 ? 0 : (id >= rows_in_table ? rows_in_table - 1 : id);
    const T* src = table + (size_t)id * width;
    T* dst = out + (size_t)r * width;
    constexpr int VEC = 16 / sizeof(T);
    if (width % VEC == 0) {
        const uint4* s4 = reinterpret_cast<const uint4*>(src);
        uint4* d4 = reinterpret_cast<uint4*>(dst);
        for (int i = threadIdx.x; i < width / VEC; i += blockDim.x) d4[i] = s4[i];
    } else {
        for (int i = threadIdx.x; i < width; i += blockDim.x) dst[i] = src[i];
    }
}

TK_API int tk_gather_rows_select(const void* table, const int* ids_host, const int* use_prev,
                                 const int* last_token, const int* slot, void* out, int rows, int width,
                                 int rows_in_table, int dtype, cudaStream_t stream) {
    TK_CHECK_ARG(rows >= 0 && width > 0 && rows_in_table > 0, "gather_rows_select: bad sizes rows=%d width=%d table=%d",
                 rows, width, rows_in_table);
    if (rows == 0) return 0;
    const int threads = width >= 1024 ? 256 : 128;
    if (dtype == TK_F32)
        tk_launch(gather_rows_select_kernel<float>, dim3(rows), dim3(threads), 0, stream, (const float*)table,
                  ids_host, use_prev, last_token, slot, (float*)out, width, rows_in_table);
    else if (dtype == TK_BF16)
        tk_launch(gather_rows_select_kernel<__nv_bfloat16>, dim3(rows), dim3(threads), 0, stream,
                  (const __nv_bfloat16*)table, ids_host, use_prev, last_token, slot, (__nv_bfloat16*)out, width,
                  rows_in_table);
    else
        TK_CHECK_ARG(false, "gather_rows_select: unknown dtype %d", dtype);
    TK_CHECK_LAUNCH("gather_rows_select");
    return 0;
}

// ---------------------------------------------------------------------------------------------
// add + RMSNorm: stream = round(residual + [prenorm](x)); y = round(round(stream*rstd) * w)
// One block per row; the row lives in shared memory as float. `x` may be a strided view.
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void add_rmsnorm_kernel(const T* x, int64_t x_stride,
                                   const T* residual, const float* __restrict__ pre_w,
                                   float pre_eps, const float* __restrict__ w, float eps,
                                   T* y, T* stream, int width) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float row[];
    __shared__ float red[33];
    const int r = blockIdx.x;
    const T* xr = x + (size_t)r * x_stride;
    float ss = 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        float v = to_f<T>(xr[i]);
        row[i] = v;
        ss += v * v;
    }
    if (pre_w != nullptr) {
        // sandwich norm on the block output before it joins the stream
        const float rstd = 1.0f / sqrtf(block_sum(ss, red) / (float)width + pre_eps);
        for (int i = threadIdx.x; i < width; i += blockDim.x)
            row[i] = round_as<T>(round_as<T>(row[i] * rstd) * pre_w[i]);
    }
    if (residual != nullptr || pre_w != nullptr) {
        ss = 0.f;
        for (int i = threadIdx.x; i < width; i += blockDim.x) {
            float v = row[i];
            if (residual != nullptr) v = round_as<T>(v + to_f<T>(residual[(size_t)r * width + i]));
            row[i] = v;
            ss += v * v;
            if (stream != nullptr) stream[(size_t)r * width + i] = from_f<T>(v);
        }
    }
    if (w == nullptr) return;  // the stream alone
    const float rstd = 1.0f / sqrtf(block_sum(ss, red) / (float)width + eps);
    for (int i = threadIdx.x; i < width; i += blockDim.x)
        y[(size_t)r * width + i] = from_f<T>(round_as<T>(row[i] * rstd) * w[i]);
}

// Fast path: the row lives in registers as 16-byte vectors (ITEMS per thread), so the kernel
// makes one trip to memory: read x (and the residual), write the stream, reduce, write y.
template <typename T, int ITEMS>
__global__ void __launch_bounds__(128)
add_rmsnorm_vec_kernel(const T* x, int64_t x_stride, const T* residual,
                       const float* __restrict__ pre_w, float pre_eps, const float* __restrict__ w,
                       float eps, T* y, T* stream, int width) {
    pdl_launch_dependents();
    pdl_wait();
    constexpr int VEC = 16 / sizeof(T);
    __shared__ float red[33];
    const int r = blockIdx.x;
    const T* xr = x + (size_t)r * x_stride;
    float v[ITEMS][VEC];
    float ss = 0.f;
    // a few rows (decode): the residual's loads go out with x's, one trip to memory for both;
    // with thousands of rows in flight the two streams are better read one after the other
    // (2,048 rows of 2,048: 7.2 us against 8.2 us)
    const bool early = residual != nullptr && gridDim.x <= 256;
    uint4 res[ITEMS];
    if (early) {
#pragma unroll
        for (int it = 0; it < ITEMS; ++it) {
            const int c = (it * 128 + threadIdx.x) * VEC;
            if (c < width) res[it] = *reinterpret_cast<const uint4*>(residual + (size_t)r * width + c);
        }
    }
#pragma unroll
    for (int it = 0; it < ITEMS; ++it) {
        const int c = (it * 128 + threadIdx.x) * VEC;
        if (c < width) {
            const uint4 raw = *reinterpret_cast<const uint4*>(xr + c);
            const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
            for (int k = 0; k < VEC; ++k) {
                v[it][k] = to_f<T>(e[k]);
                ss += v[it][k] * v[it][k];
            }
        } else {
#pragma unroll
            for (int k = 0; k < VEC; ++k) v[it][k] = 0.f;
        }
    }
    if (pre_w != nullptr) {
        const float rstd = 1.0f / sqrtf(block_sum(ss, red) / (float)width + pre_eps);
#pragma unroll
        for (int it = 0; it < ITEMS; ++it) {
            const int c = (it * 128 + threadIdx.x) * VEC;
            if (c < width) {
#pragma unroll
                for (int k = 0; k < VEC; ++k)
                    v[it][k] = round_as<T>(round_as<T>(v[it][k] * rstd) * pre_w[c + k]);
            }
        }
    }
    if (residual != nullptr || pre_w != nullptr) {
        ss = 0.f;
#pragma unroll
        for (int it = 0; it < ITEMS; ++it) {
            const int c = (it * 128 + threadIdx.x) * VEC;
            if (c < width) {
                if (residual != nullptr) {
                    if (!early) res[it] = *reinterpret_cast<const uint4*>(residual + (size_t)r * width + c);
                    const T* e = reinterpret_cast<const T*>(&res[it]);
#pragma unroll
                    for (int k = 0; k < VEC; ++k) v[it][k] = round_as<T>(v[it][k] + to_f<T>(e[k]));
                }
                uint4 packed;
                T* e = reinterpret_cast<T*>(&packed);
#pragma unroll
                for (int k = 0; k < VEC; ++k) {
                    ss += v[it][k] * v[it][k];
                    e[k] = from_f<T>(v[it][k]);
                }
                if (stream != nullptr) *reinterpret_cast<uint4*>(stream + (size_t)r * width + c) = packed;
            }
        }
    }
    if (w == nullptr) return;
    const float rstd = 1.0f / sqrtf(block_sum(ss, red) / (float)width + eps);
#pragma unroll
    for (int it = 0; it < ITEMS; ++it) {
        const int c = (it * 128 + threadIdx.x) * VEC;
        if (c < width) {
            uint4 packed;
            T* e = reinterpret_cast<T*>(&packed);
            const float4* wv = reinterpret_cast<const float4*>(w + c);
#pragma unroll
            for (int k = 0; k < VEC; k += 4) {
                const float4 ww = wv[k / 4];
                e[k] = from_f<T>(round_as<T>(v[it][k] * rstd) * ww.x);
                e[k + 1] = from_f<T>(round_as<T>(v[it][k + 1] * rstd) * ww.y);
                e[k + 2] = from_f<T>(round_as<T>(v[it][k + 2] * rstd) * ww.z);
                e[k + 3] = from_f<T>(round_as<T>(v[it][k + 3] * rstd) * ww.w);
            }
            *reinterpret_cast<uint4*>(y + (size_t)r * width + c) = packed;
        }
    }
}

template <typename T>
static bool launch_add_rmsnorm_vec(const void* x, int64_t x_stride, const void* residual,
                                   const float* pre_w, float pre_eps, const float* w, float eps,
                                   void* y, void* stream_out, int rows, int width,
                                   cudaStream_t stream) {
    constexpr int VEC = 16 / sizeof(T);
    const bool aligned = width % VEC == 0 && x_stride % VEC == 0 && (uintptr_t)x % 16 == 0 &&
                         (uintptr_t)residual % 16 == 0 && (uintptr_t)y % 16 == 0 &&
                         (uintptr_t)stream_out % 16 == 0 && (uintptr_t)w % 16 == 0;
    if (!aligned || width > 8 * 128 * VEC) return false;
    const int items = (width + 128 * VEC - 1) / (128 * VEC);
#define TK_NORM_VEC(IT)                                                                           \
    tk_launch(add_rmsnorm_vec_kernel<T, IT>, dim3(rows), dim3(128), 0, stream, (const T*)x, x_stride, (const T*)residual, \
        pre_w, pre_eps, w, eps, (T*)y, (T*)stream_out, width)
    if (items <= 1) TK_NORM_VEC(1);
    else if (items == 2) TK_NORM_VEC(2);
    else if (items <= 4) TK_NORM_VEC(4);
    else TK_NORM_VEC(8);
#undef TK_NORM_VEC
    return true;
}

TK_API int tk_add_rmsnorm(const void* x, int64_t x_stride, const void* residual,
                          const float* pre_w, float pre_eps, const float* w, float eps, void* y,
                          void* stream_out, int rows, int width, int dtype, cudaStream_t stream) {
    TK_CHECK_ARG(rows >= 0 && width > 0, "add_rmsnorm: bad sizes rows=%d width=%d", rows, width);
    TK_CHECK_ARG((size_t)width * sizeof(float) <= 200 * 1024,
                 "add_rmsnorm: width %d does not fit a row in shared memory (limit 51200)", width);
    TK_CHECK_ARG(w == nullptr || y != nullptr, "add_rmsnorm: norm weight without an output");
    if (rows == 0) return 0;
    const int threads = width >= 4096 ? 512 : (width >= 1024 ? 256 : 128);
    const size_t smem = (size_t)width * sizeof(float);
    if (dtype == TK_F32 && launch_add_rmsnorm_vec<float>(x, x_stride, residual, pre_w, pre_eps, w, eps, y,
                                                         stream_out, rows, width, stream)) {
        TK_CHECK_LAUNCH("add_rmsnorm_vec");
        return 0;
    }
    if (dtype == TK_BF16 && launch_add_rmsnorm_vec<__nv_bfloat16>(x, x_stride, residual, pre_w, pre_eps, w,
                                                                  eps, y, stream_out, rows, width, stream)) {
        TK_CHECK_LAUNCH("add_rmsnorm_vec");
        return 0;
    }
    if (dtype == TK_F32) {
        if (smem > 48 * 1024)
            cudaFuncSetAttribute(add_rmsnorm_kernel<float>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        tk_launch(add_rmsnorm_kernel<float>, dim3(rows), dim3(threads), smem, stream, 
            (const float*)x, x_stride, (const float*)residual, pre_w, pre_eps, w, eps, (float*)y,
            (float*)stream_out, width);
    } else if (dtype == TK_BF16) {
        if (smem > 48 * 1024)
            cudaFuncSetAttribute(add_rmsnorm_kernel<__nv_bfloat16>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        tk_launch(add_rmsnorm_kernel<__nv_bfloat16>, dim3(rows), dim3(threads), smem, stream, 
            (const __nv_bfloat16*)x, x_stride, (const __nv_bfloat16*)residual, pre_w, pre_eps, w, eps,
            (__nv_bfloat16*)y, (__nv_bfloat16*)stream_out, width);
    } else {
        TK_CHECK_ARG(false, "add_rmsnorm: unknown dtype %d", dtype);
    }
    TK_CHECK_LAUNCH("add_rmsnorm");
    return 0;
}

// ---------------------------------------------------------------------------------------------
// SwiGLU: out[t, i] = round(round(silu(g[t, i])) * u[t, i]) with gu = [g | u] of width 2*inter
// ---------------------------------------------------------------------------------------------
// block == 0: gu = [gate (inter) | up (inter)]; block > 0: gate and up alternate in runs of `block`
// channels (the layout the decode kernel's fused epilogue wants of the weight rows).
template <typename T>
__global__ void swiglu_kernel(const T* gu, T* out, int64_t total,
                              int inter, int block) {
    pdl_launch_dependents();
    pdl_wait();
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t step = (int64_t)gridDim.x * blockDim.x;
    for (; i < total; i += step) {
        const int64_t t = i / inter;
        const int c = (int)(i - t * inter);
        const int gi = block > 0 ? (c / block) * 2 * block + c % block : c;
        const int ui = block > 0 ? gi + block : inter + c;
        const float g = to_f<T>(gu[t * 2 * inter + gi]);
        const float u = to_f<T>(gu[t * 2 * inter + ui]);
        const float s = silu_as<T>(g);
        out[i] = from_f<T>(s * u);
    }
}

__device__ __forceinline__ float2 mul2(float2 a, float2 b) {
    float2 d;
    asm("{\n\t.reg .b64 ra, rb, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\t"
        "mul.rn.f32x2 rd, ra, rb;\n\tmov.b64 {%0, %1}, rd;\n\t}"
        : "=f"(d.x), "=f"(d.y)
        : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
    return d;
}

__device__ __forceinline__ float2 add2(float2 a, float2 b) {
    float2 d;
    asm("{\n\t.reg .b64 ra, rb, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\t"
        "add.rn.f32x2 rd, ra, rb;\n\tmov.b64 {%0, %1}, rd;\n\t}"
        : "=f"(d.x), "=f"(d.y)
        : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
    return d;
}

// 16 bytes of gate and of up per thread and step (block == 0 or block a multiple of 8 channels),
// two steps' loads in flight. One block row of the grid per token row, so no thread divides by
// the row length. The sigmoid uses the fast exponential and reciprocal: their error (a few ulp
// of a float) is far below the 16-bit rounding that follows. An earlier version with expf, a
// full-precision division and a 64-bit index division per element was instruction-bound
// (80 % issue slots busy at a third of the memory bandwidth).
__global__ void __launch_bounds__(256)
swiglu_vec_kernel(const __nv_bfloat16* gu, __nv_bfloat16* out, int rows, int inter, int block,
                  int blocks_per_row) {
    pdl_launch_dependents();
    pdl_wait();
    const int per_row = inter >> 3;
    const int t = blockIdx.x / blocks_per_row;
    const int v0 = (blockIdx.x - t * blocks_per_row) * (2 * 256) + threadIdx.x;
    const __nv_bfloat16* row = gu + (size_t)t * 2 * inter;
    uint4 graw[2], uraw[2];
    int c[2];
#pragma unroll
    for (int k = 0; k < 2; ++k) {
        const int v = v0 + k * 256;
        c[k] = v << 3;
        if (v < per_row) {
            const int gi = block > 0 ? (c[k] / block) * 2 * block + c[k] % block : c[k];
            const int ui = block > 0 ? gi + block : inter + c[k];
            graw[k] = *reinterpret_cast<const uint4*>(row + gi);
            uraw[k] = *reinterpret_cast<const uint4*>(row + ui);
        }
    }
#pragma unroll
    for (int k = 0; k < 2; ++k) {
        if (v0 + k * 256 >= per_row) continue;
        // two channels per step: packed 32-bit multiplies and adds around the exponential and the
        // reciprocal (the same operations in the same order as silu_as), one conversion to a
        // bfloat16 pair, one packed multiply with the up pair (a single rounding, as a 32-bit
        // product rounded once)
        const uint32_t* g2 = reinterpret_cast<const uint32_t*>(&graw[k]);
        const uint32_t* u2 = reinterpret_cast<const uint32_t*>(&uraw[k]);
        uint4 packed;
        uint32_t* o2 = reinterpret_cast<uint32_t*>(&packed);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 gf = make_float2(__uint_as_float(g2[e] << 16), __uint_as_float(g2[e] & 0xffff0000u));
            float2 x = mul2(gf, make_float2(TK_NEG_LOG2E, TK_NEG_LOG2E));
            x = add2(make_float2(1.0f, 1.0f), make_float2(ex2_approx(x.x), ex2_approx(x.y)));
            const float2 sl = mul2(gf, make_float2(rcp_approx(x.x), rcp_approx(x.y)));
            const __nv_bfloat162 sb = __floats2bfloat162_rn(sl.x, sl.y);
            const __nv_bfloat162 prod = __hmul2(sb, *reinterpret_cast<const __nv_bfloat162*>(&u2[e]));
            o2[e] = *reinterpret_cast<const uint32_t*>(&prod);
        }
        *reinterpret_cast<uint4*>(out + (size_t)t * inter + c[k]) = packed;
    }
}

TK_API int tk_swiglu(const void* gu, void* out, int rows, int inter, int block, int dtype,
                     cudaStream_t stream) {
    TK_CHECK_ARG(rows >= 0 && inter > 0, "swiglu: bad sizes rows=%d inter=%d", rows, inter);
    TK_CHECK_ARG(block >= 0 && (block == 0 || inter % block == 0), "swiglu: runs of %d channels do not "
                 "divide %d", block, inter);
    if (rows == 0) return 0;
    const int64_t total = (int64_t)rows * inter;
    const int threads = 256;
    if (dtype == TK_BF16 && inter % 8 == 0 && (block == 0 || block % 8 == 0) && (uintptr_t)gu % 16 == 0 &&
        (uintptr_t)out % 16 == 0) {
        const int per_row = inter / 8;
        const int blocks_per_row = (per_row + 2 * threads - 1) / (2 * threads);
        if ((int64_t)rows * blocks_per_row > 0x7fffffffLL) {
            tk_set_error("swiglu: %d rows of %d channels exceed the grid", rows, inter);
            return -1;
        }
        tk_launch(swiglu_vec_kernel, dim3((unsigned)(rows * blocks_per_row)), dim3(threads), 0, stream,
                  (const __nv_bfloat16*)gu, (__nv_bfloat16*)out, rows, inter, block, blocks_per_row);
        TK_CHECK_LAUNCH("swiglu_vec");
        return 0;
    }
    const int blocks = (int)((total + threads - 1) / threads < 148 * 16 ? (total + threads - 1) / threads
                                                                        : 148 * 16);
    if (dtype == TK_F32)
        tk_launch(swiglu_kernel<float>, dim3(blocks), dim3(threads), 0, stream, (const float*)gu, (float*)out, total, inter, block);
    else if (dtype == TK_BF16)
        tk_launch(swiglu_kernel<__nv_bfloat16>, dim3(blocks), dim3(threads), 0, stream, 
            (const __nv_bfloat16*)gu, (__nv_bfloat16*)out, total, inter, block);
    else
        TK_CHECK_ARG(false, "swiglu: unknown dtype %d", dtype);
    TK_CHECK_LAUNCH("swiglu");
    return 0;
}

// ---------------------------------------------------------------------------------------------
// per-head sigmoid gate: x[t, h, :] = round(x[t, h, :] * round(sigmoid(g[t, h])))
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void head_gate_kernel(T* x, const T* g, int64_t ldg, int64_t total, int heads,
                                 int head_dim) {
    pdl_launch_dependents();
    pdl_wait();
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t step = (int64_t)gridDim.x * blockDim.x;
    for (; i < total; i += step) {
        const int64_t th = i / head_dim;          // token * heads + head
        const float gate = to_f<T>(g[(th / heads) * ldg + th % heads]);
        const float s = round_as<T>(1.0f / (1.0f + expf(-gate)));
        x[i] = from_f<T>(to_f<T>(x[i]) * s);
    }
}

// The same on 16 bytes of bfloat16 at a time (head_dim a multiple of 8, x 16-byte aligned): a
// prompt portion's gate is a pass over [tokens, heads, head_dim], bound by memory.
__global__ void head_gate_vec_kernel(__nv_bfloat16* x, const __nv_bfloat16* g, int64_t ldg,
                                     int64_t chunks, int heads, int chunks_per_head) {
    pdl_launch_dependents();
    pdl_wait();
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t step = (int64_t)gridDim.x * blockDim.x;
    for (; i < chunks; i += step) {
        const int64_t th = i / chunks_per_head;
        const float gate = __bfloat162float(g[(th / heads) * ldg + th % heads]);
        const float s = round_as<__nv_bfloat16>(1.0f / (1.0f + expf(-gate)));
        uint4 v = reinterpret_cast<uint4*>(x)[i];
        uint32_t* w = reinterpret_cast<uint32_t*>(&v);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 f = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&w[e]));
            const __nv_bfloat162 r = __floats2bfloat162_rn(f.x * s, f.y * s);
            w[e] = *reinterpret_cast<const uint32_t*>(&r);
        }
        reinterpret_cast<uint4*>(x)[i] = v;
    }
}

// g: [rows, heads] with rows `ldg` elements apart (a column block of a wider projection's output)
TK_API int tk_head_gate(void* x, const void* g, int64_t ldg, int rows, int heads, int head_dim, int dtype,
                        cudaStream_t stream) {
    TK_CHECK_ARG(rows >= 0 && heads > 0 && head_dim > 0, "head_gate: bad sizes");
    if (rows == 0) return 0;
    const int64_t total = (int64_t)rows * heads * head_dim;
    const int threads = 256;
    const int blocks = (int)((total + threads - 1) / threads < 148 * 16 ? (total + threads - 1) / threads
                                                                        : 148 * 16);
    if (dtype == TK_BF16 && head_dim % 8 == 0 && (uintptr_t)x % 16 == 0) {
        const int64_t chunks = total / 8;
        const int vblocks = (int)((chunks + threads - 1) / threads < 148 * 16 ? (chunks + threads - 1) / threads
                                                                             : 148 * 16);
        tk_launch(head_gate_vec_kernel, dim3(vblocks), dim3(threads), 0, stream, (__nv_bfloat16*)x,
                  (const __nv_bfloat16*)g, ldg, chunks, heads, head_dim / 8);
    } else if (dtype == TK_F32)
        tk_launch(head_gate_kernel<float>, dim3(blocks), dim3(threads), 0, stream, (float*)x, (const float*)g, ldg, total, heads, head_dim);
    else if (dtype == TK_BF16)
        tk_launch(head_gate_kernel<__nv_bfloat16>, dim3(blocks), dim3(threads), 0, stream, 
            (__nv_bfloat16*)x, (const __nv_bfloat16*)g, ldg, total, heads, head_dim);
    else
        TK_CHECK_ARG(false, "head_gate: unknown dtype %d", dtype);
    TK_CHECK_LAUNCH("head_gate");
    return 0;
}

// ---------------------------------------------------------------------------------------------
// model-level options some architectures have around the layer stack: a scale on the embedding
// rows, a soft cap on the logits and a list of token ids that are never produced
// (Tokenomos models/blocks/decoder.py:167-171,185-192)
// ---------------------------------------------------------------------------------------------
// x[i] = round(x[i] * round(scale)), both roundings to the storage type
template <typename T>
__global__ void scale_rows_kernel(T* x, int64_t total, float scale) {
    pdl_launch_dependents();
    pdl_wait();
    const float s = round_as<T>(scale);
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t step = (int64_t)gridDim.x * blockDim.x;
    for (; i < total; i += step) x[i] = from_f<T>(to_f<T>(x[i]) * s);
}

TK_API int tk_scale_rows(void* x, int64_t total, float scale, int dtype, cudaStream_t stream) {
    TK_CHECK_ARG(total >= 0, "scale_rows: bad size");
    if (total == 0) return 0;
    const int threads = 256;
    const int64_t want = (total + threads - 1) / threads;
    const int blocks = (int)(want < 148 * 16 ? want : 148 * 16);
    if (dtype == TK_F32)
        tk_launch(scale_rows_kernel<float>, dim3(blocks), dim3(threads), 0, stream, (float*)x, total, scale);
    else if (dtype == TK_BF16)
        tk_launch(scale_rows_kernel<__nv_bfloat16>, dim3(blocks), dim3(threads), 0, stream, (__nv_bfloat16*)x, total, scale);
    else
        TK_CHECK_ARG(false, "scale_rows: unknown dtype %d", dtype);
    TK_CHECK_LAUNCH("scale_rows");
    return 0;
}

// logits [rows, vocab] float32, in place: cap > 0: x = cap * tanh(x / cap); then the `n_suppress`
// ids of `suppress` (each inside the vocabulary) become -inf in every row
__global__ void logit_options_kernel(float* logits, int64_t ld, int rows, int vocab, float cap,
                                     const int* suppress, int n_suppress) {
    pdl_launch_dependents();
    pdl_wait();
    const int64_t total = (int64_t)rows * vocab;
    const int64_t step = (int64_t)gridDim.x * blockDim.x;
    const float inv = cap > 0.f ? 1.0f / cap : 0.f;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += step) {
        const int col = (int)(i % vocab);
        float* at = logits + (i / vocab) * ld + col;
        bool hit = false;
        for (int k = 0; k < n_suppress; ++k) hit = hit || suppress[k] == col;
        if (hit) *at = -INFINITY;
        else if (cap > 0.f) *at = cap * tanhf(*at * inv);
    }
}

TK_API int tk_logit_options(float* logits, int64_t ld, int rows, int vocab, float cap, const int* suppress,
                            int n_suppress, cudaStream_t stream) {
    TK_CHECK_ARG(rows >= 0 && vocab > 0 && ld >= vocab && n_suppress >= 0, "logit_options: bad sizes");
    TK_CHECK_ARG(n_suppress == 0 || suppress != nullptr, "logit_options: the suppress list is missing");
    if (rows == 0 || (cap <= 0.f && n_suppress == 0)) return 0;
    const int threads = 256;
    const int64_t want = ((int64_t)rows * vocab + threads - 1) / threads;
    const int blocks = (int)(want < 148 * 16 ? want : 148 * 16);
    tk_launch(logit_options_kernel, dim3(blocks), dim3(threads), 0, stream, logits, ld, rows, vocab, cap, suppress,
              n_suppress);
    TK_CHECK_LAUNCH("logit_options");
    return 0;
}
