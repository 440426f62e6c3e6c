// Rotary position encoding in its general form, with the new keys and values written into the
// paged cache: either pairing of a head's columns (rotate-half: column i with i + R/2;
// interleaved: column 2i with 2i + 1), a table of frequencies the host computed (any scaling of
// the frequencies is in the table), a factor on cos and sin, key and value heads of different
// sizes, and values that are the keys as projected, before the rotation.
//
//   angle = float(position) * freq[i]          (32-bit; cos and sin are not rounded)
//   (u, v) -> (u cos - v sin, v cos + u sin) * 1, with cos and sin multiplied by `cs_mult`
//
// Cache layout: [pages, 2 (K|V), Hkv, P, Dp] with Dp >= max(Dk, Dv): a key fills the first Dk
// columns of its row, a value the first Dv.
#include <math.h>

#include "common.cuh"

template <typename T>
__global__ void rotary_write_kernel(const T* qkv, int64_t qkv_stride, T* q_out, T* kv_pool,
                                    const float* __restrict__ freq, float cs_mult, const int* positions,
                                    const int* tok_seq, const int* block_table, int bt_stride, int H, int Hkv,
                                    int Dk, int Dv, int Dp, int R, int P, int interleaved, int v_is_k) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float smem[];
    const int t = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    const int pos = positions[t];
    const int half = R >> 1;
    float* cs = smem;
    float* sn = smem + half;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        float s_, c_;
        sincosf((float)pos * freq[i], &s_, &c_);
        cs[i] = c_ * cs_mult;
        sn[i] = s_ * cs_mult;
    }
    __syncthreads();
    size_t cache_row = 0;
    if (Hkv > 0) {
        const int s = tok_seq[t];
        const int page = TK_PAGE(TK_K_QK_ROPE, block_table[(size_t)s * bt_stride + pos / P]);
        cache_row = (size_t)page * 2 * Hkv * P + (pos % P);
    }
    const T* row = qkv + (size_t)t * qkv_stride;
    const int v_heads = v_is_k ? 0 : Hkv;
    for (int hh = blockIdx.y * nwarp + warp; hh < H + Hkv + v_heads; hh += gridDim.y * nwarp) {
        if (hh >= H + Hkv) {                       // a value head of its own: copied
            const int kh = hh - H - Hkv;
            const T* src = row + (size_t)(H + Hkv) * Dk + (size_t)kh * Dv;
            T* dst = kv_pool + (cache_row + (size_t)(Hkv + kh) * P) * Dp;
            for (int c = lane; c < Dv; c += 32) dst[c] = src[c];
            continue;
        }
        const T* src = row + (size_t)hh * Dk;
        T* dst;
        T* copy = nullptr;
        if (hh < H) {
            dst = q_out + ((size_t)t * H + hh) * Dk;
        } else {
            const int kh = hh - H;
            dst = kv_pool + (cache_row + (size_t)kh * P) * Dp;
            if (v_is_k) copy = kv_pool + (cache_row + (size_t)(Hkv + kh) * P) * Dp;
        }
        for (int c = lane; c < Dk; c += 32) {
            const float x = to_f<T>(src[c]);
            float o = x;
            if (c < R) {
                if (interleaved) {
                    const int i = c >> 1;
                    const float y = to_f<T>(src[c ^ 1]);
                    o = (c & 1) ? x * cs[i] + y * sn[i] : x * cs[i] - y * sn[i];
                } else {
                    const bool first = c < half;
                    const int i = first ? c : c - half;
                    const float y = to_f<T>(src[first ? c + half : c - half]);
                    o = first ? x * cs[i] - y * sn[i] : x * cs[i] + y * sn[i];
                }
            }
            dst[c] = from_f<T>(o);
            if (copy != nullptr) copy[c] = src[c];
        }
    }
}

// The same, 16 bytes of bfloat16 (8 columns) per thread and step. A chunk of a rotated region
// needs its partner columns: in the interleaved layout they are in the chunk itself, in the
// rotate-half layout they are the chunk half the rotated width away, which the thread loads too.
// Needs Dk, Dv and the cache rows in whole chunks, the rotated width in whole chunks (rotate-half:
// half of it), 16-byte aligned rows.
__global__ void __launch_bounds__(128)
rotary_write_vec_kernel(const __nv_bfloat16* qkv, int64_t qkv_stride, __nv_bfloat16* q_out, __nv_bfloat16* kv_pool,
                        const float* __restrict__ freq, float cs_mult, const int* positions, const int* tok_seq,
                        const int* block_table, int bt_stride, int H, int Hkv, int Dk, int Dv, int Dp, int R,
                        int P, int interleaved, int v_is_k) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float smem[];
    const int t = blockIdx.x;
    const int pos = positions[t];
    const int half = R >> 1;
    float* cs = smem;
    float* sn = smem + half;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        float s_, c_;
        sincosf((float)pos * freq[i], &s_, &c_);
        cs[i] = c_ * cs_mult;
        sn[i] = s_ * cs_mult;
    }
    size_t cache_row = 0;
    if (Hkv > 0) {
        const int s = tok_seq[t];
        const int page = TK_PAGE(TK_K_QK_ROPE, block_table[(size_t)s * bt_stride + pos / P]);
        cache_row = (size_t)page * 2 * Hkv * P + (pos % P);
    }
    __syncthreads();
    const __nv_bfloat16* row = qkv + (size_t)t * qkv_stride;
    const int ck = Dk >> 3, cv = Dv >> 3;
    const int qk_chunks = (H + Hkv) * ck;
    const int chunks = qk_chunks + (v_is_k ? 0 : Hkv * cv);
    for (int u = blockIdx.y * blockDim.x + threadIdx.x; u < chunks; u += gridDim.y * blockDim.x) {
        if (u >= qk_chunks) {                    // a value head of its own: copied
            const int kh = (u - qk_chunks) / cv, c = ((u - qk_chunks) % cv) << 3;
            *reinterpret_cast<uint4*>(kv_pool + (cache_row + (size_t)(Hkv + kh) * P) * Dp + c) =
                *reinterpret_cast<const uint4*>(row + (size_t)(H + Hkv) * Dk + (size_t)kh * Dv + c);
            continue;
        }
        const int hh = u / ck, c = (u % ck) << 3;
        const __nv_bfloat16* src = row + (size_t)hh * Dk;
        const uint4 raw = *reinterpret_cast<const uint4*>(src + c);
        __nv_bfloat16* dst;
        if (hh < H) {
            dst = q_out + ((size_t)t * H + hh) * Dk;
        } else {
            dst = kv_pool + (cache_row + (size_t)(hh - H) * P) * Dp;
            if (v_is_k) *reinterpret_cast<uint4*>(kv_pool + (cache_row + (size_t)(Hkv + hh - H) * P) * Dp + c) = raw;
        }
        uint4 packed = raw;
        if (c < R) {
            const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(&raw);
            __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(&packed);
            if (interleaved) {
                const int i0 = c >> 1;
#pragma unroll
                for (int p = 0; p < 4; ++p) {
                    const float a = __bfloat162float(e[2 * p]), b = __bfloat162float(e[2 * p + 1]);
                    o[2 * p] = __float2bfloat16_rn(a * cs[i0 + p] - b * sn[i0 + p]);
                    o[2 * p + 1] = __float2bfloat16_rn(b * cs[i0 + p] + a * sn[i0 + p]);
                }
            } else {
                const bool first = c < half;
                const uint4 other = *reinterpret_cast<const uint4*>(src + (first ? c + half : c - half));
                const __nv_bfloat16* f = reinterpret_cast<const __nv_bfloat16*>(&other);
                const int i0 = first ? c : c - half;
#pragma unroll
                for (int p = 0; p < 8; ++p) {
                    const float a = __bfloat162float(e[p]), b = __bfloat162float(f[p]);
                    o[p] = __float2bfloat16_rn(first ? a * cs[i0 + p] - b * sn[i0 + p] : a * cs[i0 + p] + b * sn[i0 + p]);
                }
            }
        }
        *reinterpret_cast<uint4*>(dst + c) = packed;
    }
}

// qkv: rows of H query heads of Dk, Hkv key heads of Dk and (unless v_is_k) Hkv value heads of
// Dv, `qkv_stride` elements apart; q_out: [T, H, Dk]. Hkv = 0: queries only. R: rotated columns
// (even, <= Dk); freq: float [R / 2].
TK_API int tk_rotary_write(const void* qkv, int64_t qkv_stride, void* q_out, void* kv_pool, const float* freq,
                           float cs_mult, const int* positions, const int* tok_seq, const int* block_table,
                           int bt_stride, int T_, int H, int Hkv, int Dk, int Dv, int Dp, int R, int P,
                           int interleaved, int v_is_k, int dtype, cudaStream_t stream) {
    TK_CHECK_ARG(T_ >= 0 && H > 0 && Hkv >= 0 && Dk > 0 && Dv > 0 && P > 0, "rotary_write: bad sizes");
    TK_CHECK_ARG(R >= 0 && R <= Dk && R % 2 == 0, "rotary_write: %d rotated columns of a head of %d", R, Dk);
    TK_CHECK_ARG(Dp >= Dk && Dp >= Dv, "rotary_write: cache rows of %d for heads of %d and %d", Dp, Dk, Dv);
    TK_CHECK_ARG(!v_is_k || Dv == Dk, "rotary_write: values that are the keys have the keys' size");
    TK_CHECK_ARG(R <= 8192, "rotary_write: %d rotated columns above the limit of 8192", R);
    if (T_ == 0) return 0;
    const int heads = H + Hkv + (v_is_k ? 0 : Hkv);
    const int threads = 128, warps = threads / 32;
    const int per_token = T_ >= 1024 ? 1 : (heads + warps - 1) / warps;
    const size_t smem = (size_t)R * sizeof(float);
    const dim3 grid(T_, per_token);
    const bool vec = dtype == TK_BF16 && Dk % 8 == 0 && Dv % 8 == 0 && Dp % 8 == 0 && qkv_stride % 8 == 0 &&
                     R % (interleaved ? 8 : 16) == 0 && (uintptr_t)qkv % 16 == 0 && (uintptr_t)q_out % 16 == 0 &&
                     (uintptr_t)kv_pool % 16 == 0;
    if (vec) {
        const int chunks = (H + Hkv) * (Dk / 8) + (v_is_k ? 0 : Hkv * (Dv / 8));
        const dim3 vgrid(T_, T_ >= 1024 ? 1 : (chunks + threads - 1) / threads);
        tk_launch(rotary_write_vec_kernel, vgrid, dim3(threads), smem, stream, (const __nv_bfloat16*)qkv, qkv_stride,
                  (__nv_bfloat16*)q_out, (__nv_bfloat16*)kv_pool, freq, cs_mult, positions, tok_seq, block_table,
                  bt_stride, H, Hkv, Dk, Dv, Dp, R, P, interleaved, v_is_k);
        TK_CHECK_LAUNCH("rotary_write_vec");
        return 0;
    }
    if (dtype == TK_F32)
        tk_launch(rotary_write_kernel<float>, grid, dim3(threads), smem, stream, (const float*)qkv, qkv_stride,
                  (float*)q_out, (float*)kv_pool, freq, cs_mult, positions, tok_seq, block_table, bt_stride, H, Hkv,
                  Dk, Dv, Dp, R, P, interleaved, v_is_k);
    else if (dtype == TK_BF16)
        tk_launch(rotary_write_kernel<__nv_bfloat16>, grid, dim3(threads), smem, stream, (const __nv_bfloat16*)qkv,
                  qkv_stride, (__nv_bfloat16*)q_out, (__nv_bfloat16*)kv_pool, freq, cs_mult, positions, tok_seq,
                  block_table, bt_stride, H, Hkv, Dk, Dv, Dp, R, P, interleaved, v_is_k);
    else
        TK_CHECK_ARG(false, "rotary_write: unknown dtype %d", dtype);
    TK_CHECK_LAUNCH("rotary_write");
    return 0;
}
