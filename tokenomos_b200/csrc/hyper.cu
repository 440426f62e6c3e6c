// Kernels for models that carry several copies of the residual stream (hyper-connections), a
// hashed bigram embedding, and a short causal convolution on what a sublayer reads.
//
// The streams are one float32 tensor [tokens, S, width]; every sum, statistic and product here is
// 32-bit, outputs in the storage type T are rounded once.
//
//   embedding:  e = rmsnorm(table[id] + bigram[(prev * a + id * b) mod buckets]) * w, written S times;
//               the first token of a sequence takes row `buckets`; the id of a portion's last token
//               is kept per request (a state row of one int32).
//   connection: x'_t = sum_s mix[s, t] x_s + out[t] * y        (the sublayer before, if any)
//               u = sum_s in[s] x'_s;  h = u * rsqrt(mean(u^2) + eps) * w
//   input conv: o_t = h_t + sum_j taps[:, j] * h_(t - K + 1 + j), zeros before a sequence's start;
//               the last K - 1 rows of h are kept per request.
#include <math.h>

#include "common.cuh"

namespace {
constexpr int MAX_STREAMS = 8;
constexpr int MAX_TAPS = 8;
enum : int { TK_K_HYPER = 7 };
}  // namespace

// ---------------------------------------------------------------------------------------------
// hashed bigram embedding + norm, one block per token
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
embed_bigram_norm_kernel(const T* __restrict__ table, const T* __restrict__ bigram,
                         const float* __restrict__ norm_w, float eps, const int* ids, const int* use_prev,
                         const int* last_token, const int* tok_slot, const int* tok_seq, const int* cu_seqlens,
                         const int* seq_ctx, const int* seq_slot, int* prev_state, float* out, int copies,
                         int width, int vocab, int buckets, long long mul_prev, long long mul_cur) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float row[];
    __shared__ float red[33];
    __shared__ int ids_s[2];
    const int t = blockIdx.x;
    if (threadIdx.x == 0) {
        auto id_of = [&](int tt) {
            int id = (use_prev != nullptr && use_prev[tt]) ? last_token[tok_slot[tt]] : ids[tt];
            id = TK_ROW(TK_K_HYPER, id, vocab);
            return id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
        };
        const int s = tok_seq[t];
        const int first = cu_seqlens[s];
        const int id = id_of(t);
        int brow = buckets;                          // a sequence's first token
        if (bigram != nullptr) {
            int prev = -1;
            if (t > first) prev = id_of(t - 1);
            else if (seq_ctx[s] > 0) prev = prev_state[TK_SLOT(TK_K_HYPER, seq_slot[s])];
            if (prev >= 0) brow = (int)(((long long)prev * mul_prev + (long long)id * mul_cur) % (long long)buckets);
            // the block of a portion's first token has read the state; it alone writes it
            if (t == first) prev_state[TK_SLOT(TK_K_HYPER, seq_slot[s])] = id_of(cu_seqlens[s + 1] - 1);
        }
        ids_s[0] = id;
        ids_s[1] = brow;
    }
    __syncthreads();
    const T* e = table + (size_t)ids_s[0] * width;
    const T* b = bigram != nullptr ? bigram + (size_t)ids_s[1] * width : nullptr;
    float ss = 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        float v = to_f<T>(e[i]);
        if (b != nullptr) v += to_f<T>(b[i]);
        row[i] = v;
        ss += v * v;
    }
    const float rstd = 1.0f / sqrtf(block_sum(ss, red) / (float)width + eps);
    float* dst = out + (size_t)t * copies * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float v = norm_w != nullptr ? row[i] * rstd * norm_w[i] : row[i];
        for (int c = 0; c < copies; ++c) dst[(size_t)c * width + i] = v;
    }
}

TK_API int tk_embed_bigram_norm(const void* table, const void* bigram, const float* norm_w, float eps,
                                const int* ids, const int* use_prev, const int* last_token,
                                const int* tok_slot, const int* tok_seq, const int* cu_seqlens,
                                const int* seq_ctx, const int* seq_slot, int* prev_state, float* out,
                                int tokens, int copies, int width, int vocab, int buckets, int mul_prev,
                                int mul_cur, int dtype, cudaStream_t stream) {
    TK_CHECK_ARG(tokens >= 0 && copies >= 1 && width > 0 && vocab > 0, "embed: bad sizes");
    TK_CHECK_ARG(bigram == nullptr || (buckets > 0 && prev_state != nullptr), "embed: a bigram table needs buckets and a state");
    TK_CHECK_ARG((size_t)width * 4 <= 200 * 1024, "embed: a width of %d does not fit shared memory", width);
    if (tokens == 0) return 0;
    const size_t smem = (size_t)width * sizeof(float);
#define TK_EMBED(TT)                                                                                           \
    do {                                                                                                       \
        cudaFuncSetAttribute(embed_bigram_norm_kernel<TT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        tk_launch(embed_bigram_norm_kernel<TT>, dim3(tokens), dim3(256), smem, stream, (const TT*)table,        \
                  (const TT*)bigram, norm_w, eps, ids, use_prev, last_token, tok_slot, tok_seq, cu_seqlens,    \
                  seq_ctx, seq_slot, prev_state, out, copies, width, vocab, buckets, (long long)mul_prev,      \
                  (long long)mul_cur);                                                                         \
    } while (0)
    if (dtype == TK_F32) TK_EMBED(float);
    else if (dtype == TK_BF16) TK_EMBED(__nv_bfloat16);
    else TK_CHECK_ARG(false, "embed: unknown dtype %d", dtype);
#undef TK_EMBED
    TK_CHECK_LAUNCH("embed_bigram_norm");
    return 0;
}

// ---------------------------------------------------------------------------------------------
// connection write (of the sublayer before) + read + norm, one block per token.
// streams [tokens, S, width] float32, updated in place when y is given. h_out: float32 (`h32`, for
// the input convolution that follows) or T.
// ---------------------------------------------------------------------------------------------
template <typename T, bool VEC>
__global__ void __launch_bounds__(256)
hc_mix_norm_kernel(float* streams, const T* y, int64_t y_stride, const float* __restrict__ mix,
                   const float* __restrict__ out_w, const float* __restrict__ in_w,
                   const float* __restrict__ norm_w, float eps, float* h32, T* h16, int S, int width,
                   const float* __restrict__ taps, float* state, const int* seq_ctx, const int* seq_slot, int K) {
    pdl_launch_dependents();
    extern __shared__ float u_s[];
    __shared__ float red[33];
    __shared__ float c_mix[MAX_STREAMS * MAX_STREAMS], c_out[MAX_STREAMS], c_in[MAX_STREAMS];
    if (threadIdx.x < S * S) c_mix[threadIdx.x] = mix != nullptr ? mix[threadIdx.x] : (threadIdx.x / S == threadIdx.x % S ? 1.f : 0.f);
    if (threadIdx.x < S) {
        c_out[threadIdx.x] = out_w != nullptr ? out_w[threadIdx.x] : 1.f;
        c_in[threadIdx.x] = in_w != nullptr ? in_w[threadIdx.x] : 1.f;
    }
    pdl_wait();
    __syncthreads();
    const size_t t = blockIdx.x;
    float* xs = streams + t * S * width;
    float ss = 0.f;
    // a step of single tokens with the input convolution inside: the state's rows are asked for
    // first, so that they travel while the streams are summed
    float* old_s = u_s + width;                 // [K - 1][width]
    float* st = nullptr;
    if (taps != nullptr && K > 1) {
        const int ctx = seq_ctx[t];
        st = state + (size_t)TK_SLOT(TK_K_HYPER, seq_slot[t]) * (K - 1) * width;
        // (all of a thread's loads are asked for before the first is used; rows of positions before
        // the sequence's start read as zeros)
        if constexpr (VEC) {
            for (int i = threadIdx.x * 4; i < width; i += blockDim.x * 4) {
                float4 tmp[MAX_TAPS - 1];
#pragma unroll
                for (int r = 0; r < MAX_TAPS - 1; ++r)
                    if (r < K - 1)
                        tmp[r] = ctx - (K - 1) + r >= 0 ? *reinterpret_cast<const float4*>(st + (size_t)r * width + i)
                                                        : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int r = 0; r < MAX_TAPS - 1; ++r)
                    if (r < K - 1) *reinterpret_cast<float4*>(old_s + r * width + i) = tmp[r];
            }
        } else {
            for (int i = threadIdx.x; i < width; i += blockDim.x) {
                float tmp[MAX_TAPS - 1];
#pragma unroll
                for (int r = 0; r < MAX_TAPS - 1; ++r)
                    if (r < K - 1) tmp[r] = ctx - (K - 1) + r >= 0 ? st[(size_t)r * width + i] : 0.f;
#pragma unroll
                for (int r = 0; r < MAX_TAPS - 1; ++r)
                    if (r < K - 1) old_s[r * width + i] = tmp[r];
            }
        }
    }
    if constexpr (VEC) {
        for (int i = threadIdx.x * 4; i < width; i += blockDim.x * 4) {
            float4 x[MAX_STREAMS];
#pragma unroll
            for (int s = 0; s < MAX_STREAMS; ++s)
                if (s < S) x[s] = *reinterpret_cast<const float4*>(xs + (size_t)s * width + i);
            float4 u = make_float4(0.f, 0.f, 0.f, 0.f);
            if (y != nullptr) {
                float4 yv;
                if constexpr (sizeof(T) == 2) {
                    const uint2 raw = *reinterpret_cast<const uint2*>(y + t * y_stride + i);
                    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
                    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
                    yv = make_float4(a.x, a.y, b.x, b.y);
                } else {
                    yv = *reinterpret_cast<const float4*>(y + t * y_stride + i);
                }
#pragma unroll
                for (int to = 0; to < MAX_STREAMS; ++to) {
                    if (to >= S) break;
                    float4 n = make_float4(c_out[to] * yv.x, c_out[to] * yv.y, c_out[to] * yv.z, c_out[to] * yv.w);
#pragma unroll
                    for (int s = 0; s < MAX_STREAMS; ++s) {
                        if (s >= S) break;
                        const float m = c_mix[s * S + to];
                        n.x = fmaf(m, x[s].x, n.x); n.y = fmaf(m, x[s].y, n.y);
                        n.z = fmaf(m, x[s].z, n.z); n.w = fmaf(m, x[s].w, n.w);
                    }
                    *reinterpret_cast<float4*>(xs + (size_t)to * width + i) = n;
                    u.x = fmaf(c_in[to], n.x, u.x); u.y = fmaf(c_in[to], n.y, u.y);
                    u.z = fmaf(c_in[to], n.z, u.z); u.w = fmaf(c_in[to], n.w, u.w);
                }
            } else {
#pragma unroll
                for (int s = 0; s < MAX_STREAMS; ++s) {
                    if (s >= S) break;
                    u.x = fmaf(c_in[s], x[s].x, u.x); u.y = fmaf(c_in[s], x[s].y, u.y);
                    u.z = fmaf(c_in[s], x[s].z, u.z); u.w = fmaf(c_in[s], x[s].w, u.w);
                }
            }
            *reinterpret_cast<float4*>(u_s + i) = u;
            ss += u.x * u.x + u.y * u.y + u.z * u.z + u.w * u.w;
        }
    } else {
        for (int i = threadIdx.x; i < width; i += blockDim.x) {
            float x[MAX_STREAMS];
#pragma unroll
            for (int s = 0; s < MAX_STREAMS; ++s)
                if (s < S) x[s] = xs[(size_t)s * width + i];
            float u = 0.f;
            if (y != nullptr) {
                const float yv = to_f<T>(y[t * y_stride + i]);
#pragma unroll
                for (int to = 0; to < MAX_STREAMS; ++to) {
                    if (to >= S) break;
                    float n = c_out[to] * yv;
#pragma unroll
                    for (int s = 0; s < MAX_STREAMS; ++s)
                        if (s < S) n = fmaf(c_mix[s * S + to], x[s], n);
                    xs[(size_t)to * width + i] = n;
                    u = fmaf(c_in[to], n, u);
                }
            } else {
#pragma unroll
                for (int s = 0; s < MAX_STREAMS; ++s)
                    if (s < S) u = fmaf(c_in[s], x[s], u);
            }
            u_s[i] = u;
            ss += u * u;
        }
    }
    if (norm_w == nullptr) return;
    const float rstd = 1.0f / sqrtf(block_sum(ss, red) / (float)width + eps);
    if (taps != nullptr) {
        // row t is sequence t's only token; rows of the state: positions ctx - (K - 1) .. ctx - 1
        // (old_s was filled before the sum's barriers)
        for (int i = threadIdx.x; i < width; i += blockDim.x) {
            const float v = u_s[i] * rstd * norm_w[i];
            const float* w = taps + (size_t)i * K;
            float acc = v + w[K - 1] * v;
            for (int r = 0; r < K - 1; ++r) acc = fmaf(w[r], old_s[r * width + i], acc);
            h16[t * width + i] = from_f<T>(acc);
            for (int r = 0; r < K - 2; ++r) st[(size_t)r * width + i] = old_s[(r + 1) * width + i];
            if (K > 1) st[(size_t)(K - 2) * width + i] = v;
        }
        return;
    }
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float v = u_s[i] * rstd * norm_w[i];
        if (h32 != nullptr) h32[t * width + i] = v;
        else h16[t * width + i] = from_f<T>(v);
    }
}

TK_API int tk_hc_mix_norm(float* streams, const void* y, int64_t y_stride, const float* mix,
                          const float* out_w, const float* in_w, const float* norm_w, float eps,
                          float* h32, void* h16, int tokens, int S, int width, int dtype,
                          const float* taps, float* state, const int* seq_ctx, const int* seq_slot, int K,
                          cudaStream_t stream) {
    TK_CHECK_ARG(tokens >= 0 && width > 0, "hc_mix_norm: bad sizes");
    TK_CHECK_ARG(taps == nullptr || (K >= 1 && K <= MAX_TAPS && h16 != nullptr && norm_w != nullptr && seq_ctx != nullptr &&
                                     seq_slot != nullptr && (K == 1 || state != nullptr)),
                 "hc_mix_norm: the input convolution of a step of single tokens needs 1..%d taps, a state and an output", MAX_TAPS);
    TK_CHECK_ARG(S >= 1 && S <= MAX_STREAMS, "hc_mix_norm: %d streams; 1..%d are built", S, MAX_STREAMS);
    TK_CHECK_ARG((size_t)width * 4 <= 200 * 1024, "hc_mix_norm: a width of %d does not fit shared memory", width);
    TK_CHECK_ARG(norm_w == nullptr || h32 != nullptr || h16 != nullptr, "hc_mix_norm: a norm needs an output");
    if (tokens == 0) return 0;
    const size_t smem = (size_t)width * sizeof(float) * (taps != nullptr ? K : 1);
    TK_CHECK_ARG(smem <= 200 * 1024, "hc_mix_norm: %d taps of width %d do not fit shared memory", K, width);
    const bool vec = width % 4 == 0 && (y == nullptr || (y_stride % 4 == 0 && ((uintptr_t)y % 16) == 0)) &&
                     ((uintptr_t)streams % 16) == 0;
#define TK_HC(TT, V)                                                                                          \
    do {                                                                                                      \
        cudaFuncSetAttribute(hc_mix_norm_kernel<TT, V>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        tk_launch(hc_mix_norm_kernel<TT, V>, dim3(tokens), dim3(256), smem, stream, streams, (const TT*)y,     \
                  y_stride, mix, out_w, in_w, norm_w, eps, h32, (TT*)h16, S, width, taps, state, seq_ctx,      \
                  seq_slot, K);                                                                                \
    } while (0)
    if (dtype == TK_F32) { if (vec) TK_HC(float, true); else TK_HC(float, false); }
    else if (dtype == TK_BF16) { if (vec) TK_HC(__nv_bfloat16, true); else TK_HC(__nv_bfloat16, false); }
    else TK_CHECK_ARG(false, "hc_mix_norm: unknown dtype %d", dtype);
#undef TK_HC
    TK_CHECK_LAUNCH("hc_mix_norm");
    return 0;
}

// ---------------------------------------------------------------------------------------------
// input convolution with its state. One block per (tile of consecutive tokens of one sequence,
// 256 channels); a thread walks its tile's tokens with the last K - 1 rows in registers. Only the
// tile at offset 0 of a portion reads the state, and it alone writes it, after reading: tiles are
// at least K - 1 tokens long, so no later tile needs the state.
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
canon_conv_kernel(const float* h, const float* __restrict__ taps, float* state, const int* cu_seqlens,
                  const int* seq_ctx, const int* seq_slot, const int* tile_seq, const int* tile_tok0,
                  const int* tile_off, const int* tile_n, T* out, int K, int width) {
    pdl_launch_dependents();
    pdl_wait();
    const int n = tile_n[blockIdx.x];
    if (n <= 0) return;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= width) return;
    const int s = tile_seq[blockIdx.x], tok0 = tile_tok0[blockIdx.x], off = tile_off[blockIdx.x];
    const int ctx = seq_ctx[s];
    const int pos0 = ctx + off;                       // position of the tile's first token
    float w[MAX_TAPS], past[MAX_TAPS];                // past[d - 1]: the input d positions back
#pragma unroll
    for (int j = 0; j < MAX_TAPS; ++j) w[j] = j < K ? taps[(size_t)c * K + j] : 0.f;
    float* st = state != nullptr ? state + (size_t)TK_SLOT(TK_K_HYPER, seq_slot[s]) * (K - 1) * width + c : nullptr;
    float old[MAX_TAPS];                              // the state as it was (offset-0 tiles)
#pragma unroll
    for (int r = 0; r < MAX_TAPS - 1; ++r) old[r] = 0.f;
    if (off == 0 && ctx > 0) {
#pragma unroll
        for (int r = 0; r < MAX_TAPS - 1; ++r)
            if (r < K - 1) old[r] = st[(size_t)r * width];       // row r: position ctx - (K - 1) + r
    }
#pragma unroll
    for (int d = 1; d < MAX_TAPS; ++d) {
        float v = 0.f;
        if (d < K && pos0 - d >= 0) {
            if (off - d >= 0) v = h[(size_t)(tok0 - d) * width + c];
            else v = old[K - 1 - d];                  // off == 0 (tiles are >= K - 1 long) and ctx > 0
        }
        past[d - 1] = v;
    }
    for (int i = 0; i < n; ++i) {
        const float cur = h[(size_t)(tok0 + i) * width + c];
        float acc = cur + w[K - 1] * cur;
#pragma unroll
        for (int d = 1; d < MAX_TAPS; ++d)
            if (d < K) acc = fmaf(w[K - 1 - d], past[d - 1], acc);
        out[(size_t)(tok0 + i) * width + c] = from_f<T>(acc);
#pragma unroll
        for (int d = MAX_TAPS - 1; d >= 2; --d) past[d - 1] = past[d - 2];
        past[0] = cur;
    }
    if (off == 0 && st != nullptr) {
        const int first = cu_seqlens[s], len = cu_seqlens[s + 1] - first;
        // row r of the new state: position ctx + len - (K - 1) + r
#pragma unroll
        for (int r = 0; r < MAX_TAPS - 1; ++r) {
            if (r >= K - 1) break;
            const int p = len - (K - 1) + r;          // relative to the portion's first token
            float v = 0.f;
            if (p >= 0) v = h[(size_t)(first + p) * width + c];
            else if (ctx + p >= 0) v = old[r + len];  // old row of position ctx + p
            st[(size_t)r * width] = v;
        }
    }
}

TK_API int tk_canon_conv(const float* h, const float* taps, float* state, const int* cu_seqlens,
                         const int* seq_ctx, const int* seq_slot, const int* tile_seq, const int* tile_tok0,
                         const int* tile_off, const int* tile_n, int n_tiles, void* out, int K, int width,
                         int dtype, cudaStream_t stream) {
    TK_CHECK_ARG(K >= 1 && K <= MAX_TAPS, "input conv: %d taps; 1..%d are built", K, MAX_TAPS);
    TK_CHECK_ARG(K == 1 || state != nullptr, "input conv: %d taps need a state", K);
    TK_CHECK_ARG(width > 0 && n_tiles >= 0, "input conv: bad sizes");
    if (n_tiles == 0) return 0;
    dim3 grid(n_tiles, (width + 255) / 256);
    if (dtype == TK_F32)
        tk_launch(canon_conv_kernel<float>, grid, dim3(256), 0, stream, h, taps, state, cu_seqlens, seq_ctx,
                  seq_slot, tile_seq, tile_tok0, tile_off, tile_n, (float*)out, K, width);
    else if (dtype == TK_BF16)
        tk_launch(canon_conv_kernel<__nv_bfloat16>, grid, dim3(256), 0, stream, h, taps, state, cu_seqlens,
                  seq_ctx, seq_slot, tile_seq, tile_tok0, tile_off, tile_n, (__nv_bfloat16*)out, K, width);
    else
        TK_CHECK_ARG(false, "input conv: unknown dtype %d", dtype);
    TK_CHECK_LAUNCH("canon_conv");
    return 0;
}
