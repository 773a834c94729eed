// Token sampling, one block per row, every parameter per row.
//
// temperature <= 0: greedy, the first maximum. Otherwise x = logit / T restricted to the
// allowed set, then Gumbel-max: argmax(x + g), g = -log(-log u), u from a counter-based
// generator (Philox 4x32, 10 rounds) keyed by the request's (seed, step) with the vocabulary
// index as the counter, so a request draws the same tokens alone or in any batch.
// Allowed set: min_p keeps x >= max + log(min_p); top_k keeps the k largest and top_p the
// smallest top set whose mass reaches p of what the other filters left, both thresholds found
// by bisection on x (semantics of Tokenomos kernels/sampling/sample.py:1-11,32-114).
#include <math.h>

#include "common.cuh"

namespace {
constexpr int SAMPLE_THREADS = 512;
constexpr int BISECT_ITERS = 24;

struct Best {
    float v;
    int i;
};

__device__ __forceinline__ Best better(Best a, Best b) {
    // larger value wins; equal values: the smaller index (the first maximum)
    if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
    return a;
}

__device__ Best block_best(Best x, Best* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        Best y;
        y.v = __shfl_xor_sync(0xffffffffu, x.v, o);
        y.i = __shfl_xor_sync(0xffffffffu, x.i, o);
        x = better(x, y);
    }
    __syncthreads();
    if (lane == 0) red[warp] = x;
    __syncthreads();
    if (warp == 0) {
        Best t = lane < nwarp ? red[lane] : Best{-INFINITY, 0x7fffffff};
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            Best y;
            y.v = __shfl_xor_sync(0xffffffffu, t.v, o);
            y.i = __shfl_xor_sync(0xffffffffu, t.i, o);
            t = better(t, y);
        }
        if (lane == 0) red[32] = t;
    }
    __syncthreads();
    return red[32];
}

__device__ __forceinline__ uint32_t philox_first(uint32_t counter, uint32_t key0, uint32_t key1) {
    uint32_t c0 = counter, c1 = 0u, c2 = 0u, c3 = 0u;
#pragma unroll
    for (int r = 0; r < 10; ++r) {
        const uint32_t hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
        const uint32_t hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
        const uint32_t n0 = hi1 ^ c1 ^ key0, n2 = hi0 ^ c3 ^ key1;
        c0 = n0;
        c1 = lo1;
        c2 = n2;
        c3 = lo0;
        key0 += 0x9E3779B9u;
        key1 += 0xBB67AE85u;
    }
    return c0;
}

// Visit every logit of a row: 16-byte loads, four of them in flight per thread, when the row
// allows it (a scalar, strided loop makes every load wait for the one before it: 128 dependent
// trips to L2 for a 65,536-wide vocabulary). f(value, index) is called in increasing index order
// per thread.
template <typename F>
__device__ __forceinline__ void for_each_logit(const float* row, int V, F f) {
    if ((reinterpret_cast<uintptr_t>(row) & 15) == 0 && (V & 3) == 0) {
        const float4* r4 = reinterpret_cast<const float4*>(row);
        const int n4 = V >> 2;
        int i = threadIdx.x;
        for (; i + 3 * (int)blockDim.x < n4; i += 4 * blockDim.x) {
            float4 v[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) v[u] = r4[i + u * blockDim.x];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int base = (i + u * blockDim.x) * 4;
                f(v[u].x, base);
                f(v[u].y, base + 1);
                f(v[u].z, base + 2);
                f(v[u].w, base + 3);
            }
        }
        for (; i < n4; i += blockDim.x) {
            const float4 v = r4[i];
            f(v.x, i * 4);
            f(v.y, i * 4 + 1);
            f(v.z, i * 4 + 2);
            f(v.w, i * 4 + 3);
        }
    } else {
        for (int i = threadIdx.x; i < V; i += blockDim.x) f(row[i], i);
    }
}

// (sum of exp(x - top) over x >= thr, count of x >= thr), x = logit * inv_t
__device__ void mass_count(const float* row, int V, float inv_t, float top, float thr, float* red,
                           float* mass, float* count) {
    float acc = 0.f, cnt = 0.f;
    for_each_logit(row, V, [&](float v, int) {
        const float x = v * inv_t;
        if (x >= thr) {
            acc += expf(x - top);
            cnt += 1.f;
        }
    });
    *mass = block_sum(acc, red);
    *count = block_sum(cnt, red);
}
}  // namespace

// 0, or 1 + the first row whose logits held no finite value (all NaN or -inf): such a row has
// no best token; the kernel answers token 0 for it and records the row here, and the host reads
// the word where it reads the other kernels' error words (tk_sample_status).
__device__ int g_sample_error = 0;

__device__ __forceinline__ int valid_token(int tok, int row) {
    if (tok != 0x7fffffff) return tok;
    atomicCAS(&g_sample_error, 0, row + 1);
    return 0;
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* logits, int64_t stride, int V, const float* temp,
              const float* top_p, const int* top_k,
              const float* min_p, const int* seed,
              const int* step, int* out, const int* scatter_index, int* scatter_out) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ Best bred[33];
    __shared__ float fred[33];
    const int r = blockIdx.x;
    const float* row = logits + (size_t)r * stride;
    Best b{-INFINITY, 0x7fffffff};
    for_each_logit(row, V, [&](float v, int i) { b = better(b, Best{v, i}); });
    b = block_best(b, bred);
    const float t = temp[r];
    if (t <= 0.f) {
        if (threadIdx.x == 0) {
            const int tok = valid_token(b.i, r);
            out[r] = tok;
            if (scatter_out != nullptr) scatter_out[scatter_index[r]] = tok;
        }
        return;
    }
    const float inv_t = 1.0f / t;
    const float top = b.v * inv_t;
    float thr = -INFINITY;
    const float mp = min_p[r];
    if (mp > 0.f) thr = top + logf(mp);
    const int k = top_k[r];
    if (k > 0 && k < V) {
        float lo = thr == -INFINITY ? top - 1e4f : thr, hi = top;
        for (int it = 0; it < BISECT_ITERS; ++it) {
            const float mid = 0.5f * (lo + hi);
            float m, c;
            mass_count(row, V, inv_t, top, mid, fred, &m, &c);
            if (c >= (float)k) lo = mid; else hi = mid;
        }
        thr = lo;
    }
    const float pp = top_p[r];
    if (pp < 1.0f) {
        float z, c;
        mass_count(row, V, inv_t, top, thr, fred, &z, &c);
        float lo = thr == -INFINITY ? top - 1e4f : thr, hi = top;
        for (int it = 0; it < BISECT_ITERS; ++it) {
            const float mid = 0.5f * (lo + hi);
            float m;
            mass_count(row, V, inv_t, top, mid, fred, &m, &c);
            if (m >= pp * z) lo = mid; else hi = mid;
        }
        thr = lo;
    }
    const uint32_t key0 = (uint32_t)seed[r], key1 = (uint32_t)step[r];
    Best g{-INFINITY, 0x7fffffff};
    for_each_logit(row, V, [&](float v, int i) {
        const float x = v * inv_t;
        if (x >= thr) {
            const uint32_t bits = philox_first((uint32_t)i, key0, key1);
            const float u = ((float)(bits >> 9) + 0.5f) * (1.0f / 8388608.0f);  // in (0, 1), exact
            const float gum = -logf(-logf(u));
            g = better(g, Best{x + gum, i});
        }
    });
    g = block_best(g, bred);
    if (threadIdx.x == 0) {
        const int tok = valid_token(g.i == 0x7fffffff ? b.i : g.i, r);
        out[r] = tok;
        if (scatter_out != nullptr) scatter_out[scatter_index[r]] = tok;
    }
}

// logits: [rows, V] float with row stride `stride`; parameter arrays: [rows]; out: [rows] int32.
// scatter_out (optional): also scatter_out[scatter_index[r]] = token of row r.
TK_API int tk_sample(const float* logits, int64_t stride, int rows, int V, const float* temp,
                     const float* top_p, const int* top_k, const float* min_p, const int* seed,
                     const int* step, int* out, const int* scatter_index, int* scatter_out,
                     cudaStream_t stream) {
    TK_CHECK_ARG(rows >= 0 && V > 0 && stride >= V, "sample: bad sizes rows=%d V=%d", rows, V);
    if (rows == 0) return 0;
    tk_launch(sample_kernel, dim3(rows), dim3(SAMPLE_THREADS), 0, stream, logits, stride, V, temp, top_p, top_k, min_p,
                                                       seed, step, out, scatter_index, scatter_out);
    TK_CHECK_LAUNCH("sample");
    return 0;
}

// 0 if every sampled row since the last call had a finite logit; else 1 + the first row that had
// none. Resets the word.
TK_API int tk_sample_status() {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_sample_error, sizeof(int)) != cudaSuccess) return -1;
    if (v != 0) cudaMemcpyToSymbol(g_sample_error, &zero, sizeof(int));
    return v;
}
