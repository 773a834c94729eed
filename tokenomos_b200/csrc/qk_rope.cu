// Per-head q/k RMSNorm + rotate-half RoPE on the fused qkv projection, with the new keys and
// values written straight into the paged cache (one kernel instead of norm, rotate, write).
//
// Formulas (Tokenomos kernels/attention/qk.py:21-30,72-94; models/blocks/rope.py:33-35,51-59):
//   y = round(round(x * rstd) * w),  rstd = 1/sqrt(mean(x^2) + eps)      (q and k heads)
//   f = float(pos) * inv_freq[c mod R/2];  cos, sin rounded to the storage type
//   out[c] = y[c]*cos + rot[c]*sin,  rot[c] = -y[c + R/2] (c < R/2) else y[c - R/2]; c >= R passes
// V is neither normed nor rotated.  Cache layout: [pages, 2 (K|V), Hkv, P, D].
#include "common.cuh"

template <typename T>
__global__ void qk_norm_rope_write_kernel(
    const T* qkv, int64_t qkv_stride, T* q_out, T* kv_pool,
    const float* __restrict__ wq, const float* __restrict__ wk, float eps,
    const float* __restrict__ inv_freq, const int* positions,
    const int* tok_seq, const int* block_table, int bt_stride, int H,
    int Hkv, int D, int R, int P) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float smem[];
    const int t = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    const int head_first = blockIdx.y * nwarp + warp, head_step = gridDim.y * nwarp;
    const int pos = positions[t];
    const int half = R >> 1;
    // cos / sin of this token's angles, once per block (they do not depend on the head)
    float* cs = smem;
    float* sn = smem + half;
    float* buf = smem + 2 * half + warp * D;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        float s_, c_;
        sincosf((float)pos * inv_freq[i], &s_, &c_);
        cs[i] = round_as<T>(c_);
        sn[i] = round_as<T>(s_);
    }
    __syncthreads();
    size_t cache_row = 0;
    if (Hkv > 0) {
        const int s = tok_seq[t];
        const int page = TK_PAGE(TK_K_QK_ROPE, block_table[(size_t)s * bt_stride + pos / P]);
        cache_row = (size_t)page * 2 * Hkv * P + (pos % P);  // + (kv*Hkv + kh)*P rows
    }
    const T* row = qkv + (size_t)t * qkv_stride;
    for (int hh = head_first; hh < H + 2 * Hkv; hh += head_step) {
        const T* src = row + (size_t)hh * D;
        T* dst;
        const float* w = nullptr;
        bool rotate = true;
        if (hh < H) {
            dst = q_out + ((size_t)t * H + hh) * D;
            w = wq;
        } else if (hh < H + Hkv) {
            const int kh = hh - H;
            dst = kv_pool + (cache_row + (size_t)kh * P) * D;
            w = wk;
        } else {
            const int kh = hh - H - Hkv;
            dst = kv_pool + (cache_row + (size_t)(Hkv + kh) * P) * D;
            rotate = false;
        }
        if (!rotate) {
            for (int c = lane; c < D; c += 32) dst[c] = src[c];
            continue;
        }
        float ss = 0.f;
        for (int c = lane; c < D; c += 32) {
            const float v = to_f<T>(src[c]);
            buf[c] = v;
            ss += v * v;
        }
        if (w != nullptr) {
            ss = warp_sum(ss);
            const float rstd = 1.0f / sqrtf(ss / (float)D + eps);
            for (int c = lane; c < D; c += 32) buf[c] = round_as<T>(round_as<T>(buf[c] * rstd) * w[c]);
        }
        __syncwarp();
        for (int c = lane; c < D; c += 32) {
            float o = buf[c];
            if (c < R) {
                const int i = c < half ? c : c - half;
                const float rot = c < half ? -buf[c + half] : buf[c - half];
                o = o * cs[i] + rot * sn[i];
            }
            dst[c] = from_f<T>(o);
        }
        __syncwarp();
    }
}

// The same with 16-byte accesses: a head is spread over `lph` lanes (a power of two, 16 bytes
// each), so a warp takes 32 / lph heads at a time; the head's sum of squares and the rotation's
// partner elements move between lanes with shuffles instead of through shared memory. Needs
// D = lph * (16 / sizeof(T)) and half the rotary width a multiple of the 16-byte chunk.
template <typename T>
__global__ void qk_norm_rope_write_vec_kernel(
    const T* qkv, int64_t qkv_stride, T* q_out, T* kv_pool,
    const float* __restrict__ wq, const float* __restrict__ wk, float eps,
    const float* __restrict__ inv_freq, const int* positions,
    const int* tok_seq, const int* block_table, int bt_stride, int H,
    int Hkv, int D, int R, int P, int lph) {
    constexpr int VEC = 16 / sizeof(T);
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float smem[];
    const int t = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    const int heads = H + 2 * Hkv;
    const int hpw = 32 / lph;                      // heads a warp takes per pass
    const int sub = lane / lph, c = (lane % lph) * VEC;
    const T* row = qkv + (size_t)t * qkv_stride;
    // this thread's share of the first two passes is asked for before anything else: its trips
    // to memory run beside those for the position, the sequence and the page (a prompt portion's
    // block takes all heads of a token in two passes: no load then waits for another)
    const int h_first = (blockIdx.y * nwarp + warp) * hpw;
    const int h_step = gridDim.y * nwarp * hpw;
    uint4 raw_first = make_uint4(0u, 0u, 0u, 0u), raw_second = make_uint4(0u, 0u, 0u, 0u);
    if (h_first + sub < heads) raw_first = *reinterpret_cast<const uint4*>(row + (size_t)(h_first + sub) * D + c);
    if (h_first + h_step + sub < heads)
        raw_second = *reinterpret_cast<const uint4*>(row + (size_t)(h_first + h_step + sub) * D + c);
    const int pos = positions[t];
    const int seq_of_t = Hkv > 0 ? tok_seq[t] : 0;
    // (the page is looked up before the angles are computed, not after: its trip runs beside them)
    const int page = Hkv > 0 ? TK_PAGE(TK_K_QK_ROPE, block_table[(size_t)seq_of_t * bt_stride + pos / P]) : 0;
    const int half = R >> 1;
    float* cs = smem;
    float* sn = smem + half;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        float s_, c_;
        sincosf((float)pos * inv_freq[i], &s_, &c_);
        cs[i] = round_as<T>(c_);
        sn[i] = round_as<T>(s_);
    }
    __syncthreads();
    const size_t cache_row = Hkv > 0 ? (size_t)page * 2 * Hkv * P + (pos % P) : 0;
    const int half_lanes = half / VEC;
    // the lane that holds this chunk's partner in the rotation (itself beyond the rotary width)
    const int partner = c < half ? lane + half_lanes : (c < R ? lane - half_lanes : lane);
    for (int h0 = h_first; h0 < heads; h0 += h_step) {
        const int hh = h0 + sub;
        const bool live = hh < heads;
        uint4 raw = h0 == h_first ? raw_first : raw_second;
        if (h0 > h_first + h_step) {
            raw = make_uint4(0u, 0u, 0u, 0u);
            if (live) raw = *reinterpret_cast<const uint4*>(row + (size_t)hh * D + c);
        }
        const T* e = reinterpret_cast<const T*>(&raw);
        T* dst = nullptr;
        const float* w = nullptr;
        bool rotate = true;
        if (hh < H) {
            dst = q_out + ((size_t)t * H + hh) * D;
            w = wq;
        } else if (hh < H + Hkv) {
            dst = kv_pool + (cache_row + (size_t)(hh - H) * P) * D;
            w = wk;
        } else if (live) {
            dst = kv_pool + (cache_row + (size_t)(hh - H) * P) * D;      // V head hh - H - Hkv of [K | V]
            rotate = false;
        }
        float v[VEC];
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < VEC; ++i) {
            v[i] = to_f<T>(e[i]);
            ss += v[i] * v[i];
        }
        for (int o = lph >> 1; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        if (rotate && w != nullptr) {
            const float rstd = 1.0f / sqrtf(ss / (float)D + eps);
#pragma unroll
            for (int i = 0; i < VEC; ++i) v[i] = round_as<T>(round_as<T>(v[i] * rstd) * w[c + i]);
        }
        float pv[VEC];
#pragma unroll
        for (int i = 0; i < VEC; ++i) pv[i] = __shfl_sync(0xffffffffu, v[i], partner);
        if (!live) continue;
        uint4 packed = raw;
        if (rotate) {
            T* o = reinterpret_cast<T*>(&packed);
            const int i0 = c < half ? c : c - half;
#pragma unroll
            for (int i = 0; i < VEC; ++i) {
                float r = v[i];
                if (c < R) r = r * cs[i0 + i] + (c < half ? -pv[i] : pv[i]) * sn[i0 + i];
                o[i] = from_f<T>(r);
            }
        }
        *reinterpret_cast<uint4*>(dst + c) = packed;
    }
}

// qkv: [T, (H + 2*Hkv) * D] with row stride `qkv_stride` (elements); Hkv = 0 for a layer that
// only has queries (it reads another layer's cache). wq / wk may be null (no q/k norm).
TK_API int tk_qk_norm_rope_write(const void* qkv, int64_t qkv_stride, void* q_out, void* kv_pool,
                                 const float* wq, const float* wk, float eps,
                                 const float* inv_freq, const int* positions, const int* tok_seq,
                                 const int* block_table, int bt_stride, int T_, int H, int Hkv,
                                 int D, int R, int P, int dtype, cudaStream_t stream) {
    TK_CHECK_ARG(T_ >= 0 && H > 0 && Hkv >= 0 && D > 0 && P > 0, "qk_norm_rope_write: bad sizes");
    TK_CHECK_ARG(R >= 0 && R <= D && R % 2 == 0, "qk_norm_rope_write: rotary width %d of head %d", R, D);
    TK_CHECK_ARG(D <= 1024, "qk_norm_rope_write: head_dim %d above the limit of 1024", D);
    TK_CHECK_ARG((wq == nullptr) == (wk == nullptr) || Hkv == 0,
                 "qk_norm_rope_write: q and k norms come together");
    if (T_ == 0) return 0;
    const int heads = H + 2 * Hkv;
    const int threads = T_ >= 1024 ? 256 : 128;
    const int warps = threads / 32;
    // 16-byte path: the head is a power-of-two number of 16-byte chunks, the rotation's halves
    // are whole chunks, rows and bases are 16-byte aligned
    const int vec = dtype == TK_F32 ? 4 : 8;
    const int lph = D / vec;
    const bool vec_ok = D % vec == 0 && lph >= 1 && lph <= 32 && (lph & (lph - 1)) == 0 && (R / 2) % vec == 0 &&
                        qkv_stride % vec == 0 && (uintptr_t)qkv % 16 == 0 && (uintptr_t)q_out % 16 == 0 &&
                        (uintptr_t)kv_pool % 16 == 0;
    if (vec_ok) {
        const int per_pass = warps * (32 / lph);
        const int per_token = T_ >= 1024 ? 1 : (heads + per_pass - 1) / per_pass;
        const size_t smem = (size_t)R * sizeof(float);
        const dim3 grid(T_, per_token);
        if (dtype == TK_F32)
            tk_launch(qk_norm_rope_write_vec_kernel<float>, dim3(grid), dim3(threads), smem, stream,
                (const float*)qkv, qkv_stride, (float*)q_out, (float*)kv_pool, wq, wk, eps, inv_freq,
                positions, tok_seq, block_table, bt_stride, H, Hkv, D, R, P, lph);
        else if (dtype == TK_BF16)
            tk_launch(qk_norm_rope_write_vec_kernel<__nv_bfloat16>, dim3(grid), dim3(threads), smem, stream,
                (const __nv_bfloat16*)qkv, qkv_stride, (__nv_bfloat16*)q_out, (__nv_bfloat16*)kv_pool, wq,
                wk, eps, inv_freq, positions, tok_seq, block_table, bt_stride, H, Hkv, D, R, P, lph);
        else
            TK_CHECK_ARG(false, "qk_norm_rope_write: unknown dtype %d", dtype);
        TK_CHECK_LAUNCH("qk_norm_rope_write");
        return 0;
    }
    // one warp per head at a time; with few tokens the heads spread over more blocks so the GPU
    // fills, with many one block takes all heads of a token (the angles are computed once)
    const int per_token = T_ >= 1024 ? 1 : (heads + warps - 1) / warps;
    const size_t smem = ((size_t)R + (size_t)warps * D) * sizeof(float);
    const dim3 grid(T_, per_token);
    if (dtype == TK_F32)
        tk_launch(qk_norm_rope_write_kernel<float>, dim3(grid), dim3(threads), smem, stream, 
            (const float*)qkv, qkv_stride, (float*)q_out, (float*)kv_pool, wq, wk, eps, inv_freq,
            positions, tok_seq, block_table, bt_stride, H, Hkv, D, R, P);
    else if (dtype == TK_BF16)
        tk_launch(qk_norm_rope_write_kernel<__nv_bfloat16>, dim3(grid), dim3(threads), smem, stream, 
            (const __nv_bfloat16*)qkv, qkv_stride, (__nv_bfloat16*)q_out, (__nv_bfloat16*)kv_pool, wq,
            wk, eps, inv_freq, positions, tok_seq, block_table, bt_stride, H, Hkv, D, R, P);
    else
        TK_CHECK_ARG(false, "qk_norm_rope_write: unknown dtype %d", dtype);
    TK_CHECK_LAUNCH("qk_norm_rope_write");
    return 0;
}
