// Shared device helpers for the sm_100a kernels: storage-type conversion (float or bfloat16
// storage, 32-bit arithmetic everywhere), warp/block reductions, and the error channel that the
// extern "C" entry points use (every entry point returns 0 or a negative code and leaves a
// message that tk_last_error() hands to Python).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define TK_API extern "C" __attribute__((visibility("default")))

#include "checks.cuh"

// dtype codes shared with the Python side (ops/_lib.py)
enum TkDtype : int { TK_F32 = 0, TK_BF16 = 1 };

void tk_set_error(const char* fmt, ...);

#define TK_CHECK_ARG(cond, ...)            \
    do {                                   \
        if (!(cond)) {                     \
            tk_set_error(__VA_ARGS__);     \
            return -1;                     \
        }                                  \
    } while (0)

#define TK_CHECK_LAUNCH(name)                                                   \
    do {                                                                        \
        cudaError_t e__ = cudaGetLastError();                                   \
        if (e__ != cudaSuccess) {                                               \
            tk_set_error("%s: launch failed: %s", name, cudaGetErrorString(e__)); \
            return -2;                                                          \
        }                                                                       \
    } while (0)

template <typename T>
__device__ __forceinline__ float to_f(T v);
template <>
__device__ __forceinline__ float to_f<float>(float v) {
    return v;
}
template <>
__device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) {
    return __bfloat162float(v);
}

template <typename T>
__device__ __forceinline__ T from_f(float v);
template <>
__device__ __forceinline__ float from_f<float>(float v) {
    return v;
}
template <>
__device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) {
    return __float2bfloat16_rn(v);
}

// The value as it would read back after a store in T: the places where the 16-bit path rounds.
template <typename T>
__device__ __forceinline__ float round_as(float v) {
    return to_f<T>(from_f<T>(v));
}

// silu(g) = g * sigmoid(g), rounded as a store in T would. 16-bit storage takes the special
// function unit's exponential and reciprocal (a few ulp of a float, far below the rounding that
// follows), spelled out instruction by instruction so that the scalar form here and the packed
// form in the activation kernel give the same bits; 32-bit storage takes the accurate functions.
__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float rcp_approx(float x) {
    float y;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
constexpr float TK_NEG_LOG2E = -1.4426950408889634f;

template <typename T>
__device__ __forceinline__ float silu_as(float g) {
    if constexpr (sizeof(T) == 2)
        return round_as<T>(__fmul_rn(g, rcp_approx(__fadd_rn(1.0f, ex2_approx(__fmul_rn(g, TK_NEG_LOG2E))))));
    return g / (1.0f + expf(-g));
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result. `red` holds 33 floats.
__device__ __forceinline__ float block_sum(float v, float* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarp = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();  // `red` may still be read from an earlier call
    if (lane == 0) red[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nwarp ? red[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) red[32] = t;
    }
    __syncthreads();
    return red[32];
}

static inline int ceil_div(int a, int b) { return (a + b - 1) / b; }

// ---- programmatic dependent launch -----------------------------------------------------------
// Every kernel of this library is launched so that it may start while the kernel before it in
// the stream is still running (its blocks are scheduled as soon as the earlier kernel's blocks
// have all started), and every kernel calls pdl_wait() before it touches anything an earlier
// kernel may have written and before its own first global write. What a kernel reads that no
// kernel writes (weights) may be fetched before the wait: a decode step is a chain of ~100
// short kernels, and this hides their launch latency and overlaps weight streaming with the
// previous kernel's tail. tk_set_pdl(0) turns it off (plain stream order).
// One rule follows for the kernels' signatures: only pointers to data that no kernel ever writes
// (weights) are `const __restrict__`. Anything an earlier kernel produced must be read with
// ordinary loads after the wait: the compiler turns `const __restrict__` loads into ld.global.nc,
// and a line the read-only path cached while the producer was still running would be stale.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

bool tk_pdl_enabled();

template <typename... KArgs, typename... Args>
static inline cudaError_t tk_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                    cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = tk_pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
