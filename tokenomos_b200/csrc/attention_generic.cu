// Paged attention, generic path: any head size, group size, page size and storage type; 32-bit
// scores, softmax and accumulators. One block takes a tile of rows that share a KV head: the
// rows are (token, query head in the group) pairs, so a decode token brings its whole group and
// a prompt portion brings several tokens. Every key is read from the cache, the step's own keys
// included (the q/k kernel wrote them first). This is the path of the 32-bit model and the
// fallback of the 16-bit one.
//
// Score s = (q.k) * scale, key j visible to a query at position i iff j <= i and (no window or
// i - j < window); online softmax; P rounded to the storage type before P.V; the row sum keeps
// the unrounded values (Tokenomos kernels/attention/paged.py:67-76,150,267;
// models/blocks/attention.py:31-40,173).
#include <math.h>

#include "common.cuh"

namespace {
constexpr int BM = 16;       // rows per block
constexpr int BN = 32;       // keys per iteration
constexpr int THREADS = 128; // 8 threads per row
constexpr int MAX_D = 256;   // head sizes up to 256 (accumulator registers: MAX_D / 8 per thread)
}  // namespace

template <typename T>
__global__ void __launch_bounds__(THREADS)
attn_generic_kernel(const T* q, const T* kv_pool, T* out,
                    const int* positions, const int* tok_seq,
                    const int* block_table, int bt_stride,
                    const int* tile_tok0, const int* tile_ntok, int H,
                    int Hkv, int D, int P, int window, float scale, int heads_per_chunk) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float smem[];
    const int DP = D + 1;
    float* Qs = smem;                 // [BM][D+1]
    float* Ks = Qs + BM * DP;         // [BN][D+1]
    float* Vs = Ks + BN * DP;         // [BN][D]
    float* Ss = Vs + BN * D;          // [BM][BN+1]
    __shared__ int row_pos[BM];

    const int G = H / Hkv;
    const int chunks = (G + heads_per_chunk - 1) / heads_per_chunk;
    const int kvh = blockIdx.y / chunks;
    const int chunk = blockIdx.y % chunks;
    const int g0 = chunk * heads_per_chunk;
    const int gh = min(heads_per_chunk, G - g0);  // heads of this chunk
    const int tok0 = tile_tok0[blockIdx.x];
    const int ntok = tile_ntok[blockIdx.x];
    if (ntok <= 0) return;       // an unused entry of a fixed-length tile list (captured steps)
    const int rows = ntok * gh;
    const int seq = tok_seq[tok0];
    const int tid = threadIdx.x;

    // rows: r -> token tok0 + r / gh, head kvh*G + g0 + r % gh
    for (int i = tid; i < BM * D; i += THREADS) {
        const int r = i / D, c = i % D;
        float v = 0.f;
        if (r < rows) {
            const int t = tok0 + r / gh, h = kvh * G + g0 + r % gh;
            v = to_f<T>(q[((size_t)t * H + h) * D + c]);
        }
        Qs[r * DP + c] = v;
    }
    if (tid < BM) row_pos[tid] = tid < rows ? positions[tok0 + tid / gh] : -1;
    __syncthreads();

    const int pos_first = row_pos[0];
    const int pos_last = row_pos[rows - 1];
    const int lo = window > 0 ? max(0, pos_first - window + 1) : 0;

    const int r = tid >> 3;   // my row
    const int sub = tid & 7;  // my lane within the row
    const int my_pos = row_pos[r];
    float m_i = -INFINITY, l_i = 0.f;
    float acc[MAX_D / 8];
#pragma unroll
    for (int k = 0; k < MAX_D / 8; ++k) acc[k] = 0.f;

    for (int j0 = lo; j0 <= pos_last; j0 += BN) {
        // load BN keys and values: 4 threads per key
        {
            const int kk = tid >> 2, part = tid & 3;
            const int j = j0 + kk;
            if (j <= pos_last) {
                const int page = TK_PAGE(TK_K_ATTN_GENERIC, block_table[(size_t)seq * bt_stride + j / P]);
                const size_t base = ((size_t)page * 2 * Hkv * P + (size_t)kvh * P + (j % P)) * D;
                const size_t vbase = base + (size_t)Hkv * P * D;
                for (int c = part; c < D; c += 4) {
                    Ks[kk * DP + c] = to_f<T>(kv_pool[base + c]);
                    Vs[kk * D + c] = to_f<T>(kv_pool[vbase + c]);
                }
            } else {
                for (int c = part; c < D; c += 4) {
                    Ks[kk * DP + c] = 0.f;
                    Vs[kk * D + c] = 0.f;
                }
            }
        }
        __syncthreads();
        // scores of my row against keys sub, sub+8, sub+16, sub+24
        float s[4];
        float mx = -INFINITY;
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) {
            const int kk = sub + 8 * jj;
            const int j = j0 + kk;
            float d = 0.f;
            const float* qr = Qs + r * DP;
            const float* kr = Ks + kk * DP;
            for (int c = 0; c < D; ++c) d += qr[c] * kr[c];
            d *= scale;
            const bool visible = my_pos >= 0 && j <= my_pos && (window <= 0 || my_pos - j < window);
            s[jj] = visible ? d : -INFINITY;
            mx = fmaxf(mx, s[jj]);
        }
        // row maximum over the 8 threads of the row (they are 8 neighbouring lanes)
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
        const float m_new = fmaxf(m_i, mx);
        const float m_safe = m_new == -INFINITY ? 0.f : m_new;
        const float alpha = expf(m_i - m_safe);
        float psum = 0.f;
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) {
            const float p = expf(s[jj] - m_safe);
            psum += p;
            Ss[r * (BN + 1) + sub + 8 * jj] = round_as<T>(p);
        }
        psum += __shfl_xor_sync(0xffffffffu, psum, 1);
        psum += __shfl_xor_sync(0xffffffffu, psum, 2);
        psum += __shfl_xor_sync(0xffffffffu, psum, 4);
        l_i = l_i * alpha + psum;
        m_i = m_new;
        __syncthreads();
        // acc[r][c] for c = sub + 8k
        const float* pr = Ss + r * (BN + 1);
#pragma unroll
        for (int k = 0; k < MAX_D / 8; ++k) {
            const int c = sub + 8 * k;
            if (c < D) {
                float a = acc[k] * alpha;
                for (int kk = 0; kk < BN; ++kk) a += pr[kk] * Vs[kk * D + c];
                acc[k] = a;
            }
        }
        __syncthreads();
    }
    if (r < rows) {
        const int t = tok0 + r / gh, h = kvh * G + g0 + r % gh;
        const float inv = l_i > 0.f ? 1.0f / l_i : 0.f;
#pragma unroll
        for (int k = 0; k < MAX_D / 8; ++k) {
            const int c = sub + 8 * k;
            if (c < D) out[((size_t)t * H + h) * D + c] = from_f<T>(acc[k] * inv);
        }
    }
}

// Shared memory the kernel needs for head size D (bytes).
static size_t attn_generic_smem(int D) {
    return ((size_t)BM * (D + 1) + (size_t)BN * (D + 1) + (size_t)BN * D + (size_t)BM * (BN + 1)) * sizeof(float);
}

// Rows per tile this kernel takes: a tile holds `tokens_per_tile` tokens of one sequence with
// `heads_per_chunk` query heads each, tokens_per_tile * heads_per_chunk <= 16.
TK_API int tk_attn_generic_rows() { return BM; }

// q, out: [T, H, D]; kv_pool: [pages, 2, Hkv, P, D]; tiles: first token and token count of each
// tile (tokens of one sequence, consecutive positions); window <= 0: none.
TK_API int tk_attn_generic(const void* q, const void* kv_pool, void* out, const int* positions,
                           const int* tok_seq, const int* block_table, int bt_stride,
                           const int* tile_tok0, const int* tile_ntok, int n_tiles,
                           int tokens_per_tile, int H, int Hkv, int D, int P, int window,
                           float scale, int dtype, cudaStream_t stream) {
    TK_CHECK_ARG(H > 0 && Hkv > 0 && H % Hkv == 0, "attention: %d query heads over %d KV heads", H, Hkv);
    TK_CHECK_ARG(D > 0 && D <= MAX_D, "attention: head_dim %d outside 1..%d", D, MAX_D);
    TK_CHECK_ARG(P > 0 && n_tiles >= 0, "attention: bad page size or tile count");
    if (n_tiles == 0) return 0;
    const int G = H / Hkv;
    TK_CHECK_ARG(tokens_per_tile >= 1 && tokens_per_tile <= BM, "attention: %d tokens per tile", tokens_per_tile);
    const int heads_per_chunk = min(G, BM / tokens_per_tile);
    TK_CHECK_ARG(heads_per_chunk >= 1, "attention: tile of %d tokens leaves no room for a head", tokens_per_tile);
    const int chunks = (G + heads_per_chunk - 1) / heads_per_chunk;
    const size_t smem = attn_generic_smem(D);
    dim3 grid(n_tiles, Hkv * chunks);
    if (dtype == TK_F32) {
        cudaFuncSetAttribute(attn_generic_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        tk_launch(attn_generic_kernel<float>, dim3(grid), dim3(THREADS), smem, stream, 
            (const float*)q, (const float*)kv_pool, (float*)out, positions, tok_seq, block_table,
            bt_stride, tile_tok0, tile_ntok, H, Hkv, D, P, window, scale, heads_per_chunk);
    } else if (dtype == TK_BF16) {
        cudaFuncSetAttribute(attn_generic_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        tk_launch(attn_generic_kernel<__nv_bfloat16>, dim3(grid), dim3(THREADS), smem, stream, 
            (const __nv_bfloat16*)q, (const __nv_bfloat16*)kv_pool, (__nv_bfloat16*)out, positions,
            tok_seq, block_table, bt_stride, tile_tok0, tile_ntok, H, Hkv, D, P, window, scale,
            heads_per_chunk);
    } else {
        TK_CHECK_ARG(false, "attention: unknown dtype %d", dtype);
    }
    TK_CHECK_LAUNCH("attn_generic");
    return 0;
}
