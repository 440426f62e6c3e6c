// Attention over a cache of latents: every position keeps one row [c (R) | k_rot (Dr)], the
// normed key/value latent and one rotated key part that all heads share. With the keys'
// up-projection taken into the queries (q_lat[h] = W_uk[h]^T q[h]) a head's score is
// (q_lat . c + q_rot . k_rot) * scale and its output, before the values' up-projection, is
// sum_j p_j c_j: attention with one key/value head whose key is the whole row and whose value
// is the row's first R columns.
//
//   prepare: c_q = rmsnorm(row[0:Rq]) * wq;  c = rmsnorm(row[Rq:Rq+R]) * wkv -> cache;
//            k_rot = rotate(row[Rq+R : Rq+R+Dr]) -> cache      (interleaved pairs, 32-bit angles)
//   rotate_q: the last Dr columns of every query head, in place
//   attention: 32-bit scores, softmax and sums; storage float or bfloat16
#include <math.h>

#include "common.cuh"

namespace {
enum : int { TK_K_LATENT = 8 };
constexpr int BM = 16;       // rows (token x head) per block
constexpr int BN = 32;       // keys per iteration
constexpr int THREADS = 128; // 8 threads per row
}  // namespace

// (u, v) at columns (2i, 2i + 1), i < rot / 2, turned by pos * freq[i]; other columns unchanged
template <typename T>
__device__ __forceinline__ float rotated(const T* src, int c, int rot, const float* cs, const float* sn) {
    const float x = to_f<T>(src[c]);
    if (c >= rot) return x;
    const int i = c >> 1;
    const float y = to_f<T>(src[c ^ 1]);
    return (c & 1) ? x * cs[i] + y * sn[i] : x * cs[i] - y * sn[i];
}

template <typename T>
__global__ void __launch_bounds__(256)
latent_prepare_kernel(const T* proj, int64_t proj_stride, const float* __restrict__ wq,
                      const float* __restrict__ wkv, float eps, const float* __restrict__ freq,
                      const int* positions, const int* tok_seq, const int* block_table, int bt_stride,
                      T* cq_out, T* cache, int Rq, int R, int Dr, int rot, int P) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float smem[];
    __shared__ float red[33];
    float* cs = smem;
    float* sn = smem + rot / 2;
    const int t = blockIdx.x;
    const int pos = positions[t];
    for (int i = threadIdx.x; i < rot / 2; i += blockDim.x) sincosf((float)pos * freq[i], &sn[i], &cs[i]);
    const T* row = proj + (size_t)t * proj_stride;
    float ss = 0.f;
    for (int i = threadIdx.x; i < Rq; i += blockDim.x) {
        const float v = to_f<T>(row[i]);
        ss += v * v;
    }
    const float rq = Rq > 0 ? 1.0f / sqrtf(block_sum(ss, red) / (float)Rq + eps) : 0.f;
    for (int i = threadIdx.x; i < Rq; i += blockDim.x)
        cq_out[(size_t)t * Rq + i] = from_f<T>(to_f<T>(row[i]) * rq * wq[i]);
    ss = 0.f;
    for (int i = threadIdx.x; i < R; i += blockDim.x) {
        const float v = to_f<T>(row[Rq + i]);
        ss += v * v;
    }
    const float rk = 1.0f / sqrtf(block_sum(ss, red) / (float)R + eps);   // (its barriers also publish cs / sn)
    const int page = TK_PAGE(TK_K_LATENT, block_table[(size_t)tok_seq[t] * bt_stride + pos / P]);
    T* dst = cache + ((size_t)page * P + pos % P) * (R + Dr);
    for (int i = threadIdx.x; i < R; i += blockDim.x) dst[i] = from_f<T>(to_f<T>(row[Rq + i]) * rk * wkv[i]);
    for (int i = threadIdx.x; i < Dr; i += blockDim.x) dst[R + i] = from_f<T>(rotated<T>(row + Rq + R, i, rot, cs, sn));
}

TK_API int tk_latent_prepare(const void* proj, int64_t proj_stride, const float* wq, const float* wkv,
                             float eps, const float* freq, const int* positions, const int* tok_seq,
                             const int* block_table, int bt_stride, void* cq_out, void* cache, int tokens,
                             int Rq, int R, int Dr, int rot, int P, int dtype, cudaStream_t stream) {
    TK_CHECK_ARG(tokens >= 0 && Rq >= 0 && R > 0 && Dr >= 0 && P > 0, "latent_prepare: bad sizes");
    TK_CHECK_ARG(rot % 2 == 0 && rot >= 0 && rot <= Dr, "latent_prepare: %d rotated columns of %d", rot, Dr);
    if (tokens == 0) return 0;
    const size_t smem = (size_t)(rot + 2) * sizeof(float);
    if (dtype == TK_F32)
        tk_launch(latent_prepare_kernel<float>, dim3(tokens), dim3(256), smem, stream, (const float*)proj,
                  proj_stride, wq, wkv, eps, freq, positions, tok_seq, block_table, bt_stride, (float*)cq_out,
                  (float*)cache, Rq, R, Dr, rot, P);
    else if (dtype == TK_BF16)
        tk_launch(latent_prepare_kernel<__nv_bfloat16>, dim3(tokens), dim3(256), smem, stream,
                  (const __nv_bfloat16*)proj, proj_stride, wq, wkv, eps, freq, positions, tok_seq, block_table,
                  bt_stride, (__nv_bfloat16*)cq_out, (__nv_bfloat16*)cache, Rq, R, Dr, rot, P);
    else
        TK_CHECK_ARG(false, "latent_prepare: unknown dtype %d", dtype);
    TK_CHECK_LAUNCH("latent_prepare");
    return 0;
}

// q [tokens, H, D + Dr]: the last Dr columns of every head rotated in place. One block per token.
template <typename T>
__global__ void __launch_bounds__(128)
latent_rotate_q_kernel(T* q, const float* __restrict__ freq, const int* positions, int H, int D, int Dr, int rot) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float smem[];
    float* cs = smem;
    float* sn = smem + rot / 2;
    const int t = blockIdx.x;
    const int pos = positions[t];
    for (int i = threadIdx.x; i < rot / 2; i += blockDim.x) sincosf((float)pos * freq[i], &sn[i], &cs[i]);
    __syncthreads();
    // a thread takes a pair of columns, so that both are read before either is written
    const int pairs = rot / 2;
    for (int k = threadIdx.x; k < H * pairs; k += blockDim.x) {
        const int h = k / pairs, i = k % pairs;
        T* p = q + ((size_t)t * H + h) * (D + Dr) + D + 2 * i;
        const float u = to_f<T>(p[0]), v = to_f<T>(p[1]);
        p[0] = from_f<T>(u * cs[i] - v * sn[i]);
        p[1] = from_f<T>(v * cs[i] + u * sn[i]);
    }
}

TK_API int tk_latent_rotate_q(void* q, const float* freq, const int* positions, int tokens, int H, int D,
                              int Dr, int rot, int dtype, cudaStream_t stream) {
    TK_CHECK_ARG(tokens >= 0 && H > 0 && D >= 0 && Dr >= 0, "latent_rotate_q: bad sizes");
    TK_CHECK_ARG(rot % 2 == 0 && rot >= 0 && rot <= Dr, "latent_rotate_q: %d rotated columns of %d", rot, Dr);
    if (tokens == 0 || rot == 0) return 0;
    const size_t smem = (size_t)(rot + 2) * sizeof(float);
    if (dtype == TK_F32)
        tk_launch(latent_rotate_q_kernel<float>, dim3(tokens), dim3(128), smem, stream, (float*)q, freq, positions,
                  H, D, Dr, rot);
    else if (dtype == TK_BF16)
        tk_launch(latent_rotate_q_kernel<__nv_bfloat16>, dim3(tokens), dim3(128), smem, stream, (__nv_bfloat16*)q,
                  freq, positions, H, D, Dr, rot);
    else
        TK_CHECK_ARG(false, "latent_rotate_q: unknown dtype %d", dtype);
    TK_CHECK_LAUNCH("latent_rotate_q");
    return 0;
}

// ---------------------------------------------------------------------------------------------
// Attention over the latent cache, general form: any sizes, either storage type, 32-bit
// arithmetic throughout. A block takes a tile of rows (token, head): consecutive tokens of one
// sequence times a chunk of heads. Key j is visible to a query at position i iff
// 0 <= i - j < window (window <= 0: every earlier key).
//   q_lat [H, tokens, R] (row stride R),  q_rot: column D.. of q [tokens, H, D + Dr]
//   out   [H, tokens, R]
// ---------------------------------------------------------------------------------------------
template <typename T, int ACC>
__global__ void __launch_bounds__(THREADS)
attn_latent_kernel(const T* q_lat, const T* q, const T* cache, T* out, const int* positions,
                   const int* tok_seq, const int* block_table, int bt_stride, const int* tile_tok0,
                   const int* tile_ntok, int tokens, int H, int D, int R, int Dr, int P, int window,
                   float scale, int heads_per_chunk) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float smem[];
    const int DK = R + Dr, DP = DK + 1;
    float* Qs = smem;                 // [BM][DK + 1]
    float* Ks = Qs + BM * DP;         // [BN][DK + 1]
    float* Ss = Ks + BN * DP;         // [BM][BN + 1]
    __shared__ int row_pos[BM];

    const int chunk = blockIdx.y;
    const int g0 = chunk * heads_per_chunk;
    const int gh = min(heads_per_chunk, H - g0);
    const int tok0 = tile_tok0[blockIdx.x];
    const int ntok = tile_ntok[blockIdx.x];
    if (ntok <= 0) return;
    const int rows = ntok * gh;
    const int seq = tok_seq[tok0];
    const int tid = threadIdx.x;

    for (int i = tid; i < BM * DK; i += THREADS) {
        const int r = i / DK, c = i % DK;
        float v = 0.f;
        if (r < rows) {
            const int t = tok0 + r / gh, h = g0 + r % gh;
            v = c < R ? to_f<T>(q_lat[((size_t)h * tokens + t) * R + c])
                      : to_f<T>(q[((size_t)t * H + h) * (D + Dr) + D + (c - R)]);
        }
        Qs[r * DP + c] = v;
    }
    if (tid < BM) row_pos[tid] = tid < rows ? positions[tok0 + tid / gh] : -1;
    __syncthreads();

    const int pos_first = row_pos[0];
    const int pos_last = row_pos[rows - 1];
    const int lo = window > 0 ? max(0, pos_first - window + 1) : 0;
    const int r = tid >> 3, sub = tid & 7;
    const int my_pos = row_pos[r];
    float m_i = -INFINITY, l_i = 0.f;
    float acc[ACC];
#pragma unroll
    for (int k = 0; k < ACC; ++k) acc[k] = 0.f;

    const int n_it = (pos_last - lo) / BN + 1;
    for (int it = 0; it < n_it; ++it) {
        const int j0 = lo + it * BN;
        {
            const int kk = tid >> 2, part = tid & 3;
            const int j = j0 + kk;
            if (j <= pos_last) {
                const int page = TK_PAGE(TK_K_LATENT, block_table[(size_t)seq * bt_stride + j / P]);
                const T* src = cache + ((size_t)page * P + (j % P)) * DK;
                for (int c = part; c < DK; c += 4) Ks[kk * DP + c] = to_f<T>(src[c]);
            } else {
                for (int c = part; c < DK; c += 4) Ks[kk * DP + c] = 0.f;
            }
        }
        __syncthreads();
        float s[4];
        float mx = -INFINITY;
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) {
            const int kk = sub + 8 * jj;
            const int j = j0 + kk;
            float d = 0.f;
            const float* qr = Qs + r * DP;
            const float* kr = Ks + kk * DP;
            for (int c = 0; c < DK; ++c) d = fmaf(qr[c], kr[c], d);
            d *= scale;
            const bool visible = my_pos >= 0 && j <= pos_last && j <= my_pos && (window <= 0 || my_pos - j < window);
            s[jj] = visible ? d : -INFINITY;
            mx = fmaxf(mx, s[jj]);
        }
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
            Ss[r * (BN + 1) + sub + 8 * jj] = p;
        }
        psum += __shfl_xor_sync(0xffffffffu, psum, 1);
        psum += __shfl_xor_sync(0xffffffffu, psum, 2);
        psum += __shfl_xor_sync(0xffffffffu, psum, 4);
        l_i = l_i * alpha + psum;
        m_i = m_new;
        __syncthreads();
        const float* pr = Ss + r * (BN + 1);
#pragma unroll
        for (int k = 0; k < ACC; ++k) {
            const int c = sub + 8 * k;
            if (c < R) {
                float a = acc[k] * alpha;
                for (int kk = 0; kk < BN; ++kk) a = fmaf(pr[kk], Ks[kk * DP + c], a);
                acc[k] = a;
            }
        }
        __syncthreads();
    }
    if (r < rows) {
        const int t = tok0 + r / gh, h = g0 + r % gh;
        const float inv = l_i > 0.f ? 1.0f / l_i : 0.f;
#pragma unroll
        for (int k = 0; k < ACC; ++k) {
            const int c = sub + 8 * k;
            if (c < R) out[((size_t)h * tokens + t) * R + c] = from_f<T>(acc[k] * inv);
        }
    }
}

TK_API int tk_attn_latent_rows() { return BM; }
TK_API int tk_attn_latent_max_rank() { return 512; }

template <typename T, int ACC>
static int launch_attn_latent(const void* q_lat, const void* q, const void* cache, void* out, const int* positions,
                              const int* tok_seq, const int* block_table, int bt_stride, const int* tile_tok0,
                              const int* tile_ntok, int n_tiles, int tokens, int H, int D, int R, int Dr, int P,
                              int window, float scale, int heads_per_chunk, cudaStream_t stream) {
    const int DK = R + Dr;
    const size_t smem = ((size_t)(BM + BN) * (DK + 1) + (size_t)BM * (BN + 1)) * sizeof(float);
    TK_CHECK_ARG(smem <= 220 * 1024, "latent attention: rows of %d columns do not fit shared memory", DK);
    cudaFuncSetAttribute(attn_latent_kernel<T, ACC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    dim3 grid(n_tiles, (H + heads_per_chunk - 1) / heads_per_chunk);
    tk_launch(attn_latent_kernel<T, ACC>, grid, dim3(THREADS), smem, stream, (const T*)q_lat, (const T*)q,
              (const T*)cache, (T*)out, positions, tok_seq, block_table, bt_stride, tile_tok0, tile_ntok, tokens, H,
              D, R, Dr, P, window, scale, heads_per_chunk);
    return 0;
}

TK_API int tk_attn_latent(const void* q_lat, const void* q, const void* cache, void* out, const int* positions,
                          const int* tok_seq, const int* block_table, int bt_stride, const int* tile_tok0,
                          const int* tile_ntok, int n_tiles, int tokens_per_tile, int tokens, int H, int D, int R,
                          int Dr, int P, int window, float scale, int dtype, cudaStream_t stream) {
    TK_CHECK_ARG(H > 0 && R > 0 && R <= 512 && Dr >= 0 && D >= 0, "latent attention: bad sizes H=%d R=%d Dr=%d", H, R, Dr);
    TK_CHECK_ARG(P > 0 && n_tiles >= 0 && tokens >= 0, "latent attention: bad page size or counts");
    TK_CHECK_ARG(tokens_per_tile >= 1 && tokens_per_tile <= BM, "latent attention: %d tokens per tile", tokens_per_tile);
    if (n_tiles == 0) return 0;
    const int hpc = min(H, BM / tokens_per_tile);
    int rc;
#define TK_AL(TT)                                                                                                  \
    (R <= 64 ? launch_attn_latent<TT, 8>(q_lat, q, cache, out, positions, tok_seq, block_table, bt_stride, tile_tok0, \
                                        tile_ntok, n_tiles, tokens, H, D, R, Dr, P, window, scale, hpc, stream)      \
     : R <= 128 ? launch_attn_latent<TT, 16>(q_lat, q, cache, out, positions, tok_seq, block_table, bt_stride,        \
                                            tile_tok0, tile_ntok, n_tiles, tokens, H, D, R, Dr, P, window, scale,    \
                                            hpc, stream)                                                            \
     : R <= 256 ? launch_attn_latent<TT, 32>(q_lat, q, cache, out, positions, tok_seq, block_table, bt_stride,        \
                                            tile_tok0, tile_ntok, n_tiles, tokens, H, D, R, Dr, P, window, scale,    \
                                            hpc, stream)                                                            \
                : launch_attn_latent<TT, 64>(q_lat, q, cache, out, positions, tok_seq, block_table, bt_stride,        \
                                            tile_tok0, tile_ntok, n_tiles, tokens, H, D, R, Dr, P, window, scale,    \
                                            hpc, stream))
    if (dtype == TK_F32) rc = TK_AL(float);
    else if (dtype == TK_BF16) rc = TK_AL(__nv_bfloat16);
    else TK_CHECK_ARG(false, "latent attention: unknown dtype %d", dtype);
#undef TK_AL
    if (rc) return rc;
    TK_CHECK_LAUNCH("attn_latent");
    return 0;
}

// out[t, h, :] = x[h, t, :] * sigmoid(g[t, h])   (x [H, tokens, Dv] -> out [tokens, H, Dv]); g may be
// a column block of a wider row (g_stride). g null: the transposition alone.
template <typename T>
__global__ void head_gate_transpose_kernel(const T* x, const T* g, int64_t g_stride, T* out, int tokens, int H, int Dv) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t n = (size_t)tokens * H * Dv;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const int c = (int)(i % Dv);
        const size_t th = i / Dv;
        const int h = (int)(th % H);
        const size_t t = th / H;
        float v = to_f<T>(x[((size_t)h * tokens + t) * Dv + c]);
        if (g != nullptr) v *= 1.0f / (1.0f + expf(-to_f<T>(g[t * g_stride + h])));
        out[i] = from_f<T>(v);
    }
}

TK_API int tk_head_gate_transpose(const void* x, const void* g, int64_t g_stride, void* out, int tokens, int H,
                                  int Dv, int dtype, cudaStream_t stream) {
    TK_CHECK_ARG(tokens >= 0 && H > 0 && Dv > 0, "head_gate_transpose: bad sizes");
    if (tokens == 0) return 0;
    const size_t n = (size_t)tokens * H * Dv;
    const int blocks = (int)((n + 255) / 256 < (size_t)(148 * 16) ? (n + 255) / 256 : (size_t)(148 * 16));
    if (dtype == TK_F32)
        tk_launch(head_gate_transpose_kernel<float>, dim3(blocks), dim3(256), 0, stream, (const float*)x,
                  (const float*)g, g_stride, (float*)out, tokens, H, Dv);
    else if (dtype == TK_BF16)
        tk_launch(head_gate_transpose_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream,
                  (const __nv_bfloat16*)x, (const __nv_bfloat16*)g, g_stride, (__nv_bfloat16*)out, tokens, H, Dv);
    else
        TK_CHECK_ARG(false, "head_gate_transpose: unknown dtype %d", dtype);
    TK_CHECK_LAUNCH("head_gate_transpose");
    return 0;
}
