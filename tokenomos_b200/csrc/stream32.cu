// Row-wise kernels for models whose residual stream is kept in 32-bit whatever the storage type
// of the activations: the stream's adds with the RMSNorm that follows them, a clamped gated
// activation, and an element-wise sigmoid gate. Inputs and outputs of the projections around
// them are float or bfloat16 (T); every sum, statistic and product here is formed in 32-bit and
// a T output is rounded exactly once.
#include <math.h>

#include "common.cuh"

// ---------------------------------------------------------------------------------------------
// stream' = stream + x + rows + vec  (each addend optional, added in this order, 32-bit);
// y = T(stream' * rsqrt(mean(stream'^2) + eps) * w)   (w optional: without it only the adds)
// One block per row. A thread keeps its elements of the row in registers when the row is short
// enough (ITEMS per thread), else it reads its own writes back from stream_out.
// ---------------------------------------------------------------------------------------------
template <typename T, int ITEMS>
__global__ void __launch_bounds__(256)
stream32_add_norm_kernel(const float* stream_in, const T* x, int64_t x_stride, const T* rows_add,
                         const float* __restrict__ vec_add, const float* __restrict__ w, float eps,
                         float* stream_out, T* y, int width) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float red[33];
    const size_t r = blockIdx.x;
    auto sum_at = [&](int i) {
        float v = stream_in != nullptr ? stream_in[r * width + i] : 0.f;
        if (x != nullptr) v += to_f<T>(x[r * x_stride + i]);
        if (rows_add != nullptr) v += to_f<T>(rows_add[r * width + i]);
        if (vec_add != nullptr) v += vec_add[i];
        if (stream_out != nullptr) stream_out[r * width + i] = v;
        return v;
    };
    float ss = 0.f;
    if constexpr (ITEMS > 0) {
        float keep[ITEMS];
#pragma unroll
        for (int k = 0; k < ITEMS; ++k) {
            const int i = threadIdx.x + k * blockDim.x;
            keep[k] = i < width ? sum_at(i) : 0.f;
            ss += keep[k] * keep[k];
        }
        if (w == nullptr) return;
        const float rstd = 1.0f / sqrtf(block_sum(ss, red) / (float)width + eps);
#pragma unroll
        for (int k = 0; k < ITEMS; ++k) {
            const int i = threadIdx.x + k * blockDim.x;
            if (i < width) y[r * width + i] = from_f<T>(keep[k] * rstd * w[i]);
        }
    } else {
        for (int i = threadIdx.x; i < width; i += blockDim.x) {
            const float v = sum_at(i);
            ss += v * v;
        }
        if (w == nullptr) return;
        const float rstd = 1.0f / sqrtf(block_sum(ss, red) / (float)width + eps);
        for (int i = threadIdx.x; i < width; i += blockDim.x)
            y[r * width + i] = from_f<T>(stream_out[r * width + i] * rstd * w[i]);
    }
}

template <typename T>
static int launch_stream32(const float* stream_in, const void* x, int64_t x_stride, const void* rows_add,
                           const float* vec_add, const float* w, float eps, float* stream_out, void* y,
                           int rows, int width, cudaStream_t stream) {
    const int threads = width >= 1024 ? 256 : 128;
    const int per_thread = (width + threads - 1) / threads;
    if (per_thread <= 8)
        tk_launch(stream32_add_norm_kernel<T, 8>, dim3(rows), dim3(threads), 0, stream, stream_in, (const T*)x,
                  x_stride, (const T*)rows_add, vec_add, w, eps, stream_out, (T*)y, width);
    else
        tk_launch(stream32_add_norm_kernel<T, 0>, dim3(rows), dim3(threads), 0, stream, stream_in, (const T*)x,
                  x_stride, (const T*)rows_add, vec_add, w, eps, stream_out, (T*)y, width);
    return 0;
}

// stream_in / stream_out: float [rows, width] (may be the same buffer; stream_out may be null only
// when the row fits the register path, i.e. width <= 2048, and the new stream is not wanted);
// x: T rows `x_stride` elements apart; rows_add: T [rows, width]; vec_add, w: float [width].
TK_API int tk_stream32_add_norm(const float* stream_in, const void* x, int64_t x_stride, const void* rows_add,
                                const float* vec_add, const float* w, float eps, float* stream_out, void* y,
                                int rows, int width, int dtype, cudaStream_t stream) {
    TK_CHECK_ARG(rows >= 0 && width > 0, "stream32_add_norm: bad sizes rows=%d width=%d", rows, width);
    TK_CHECK_ARG(stream_in != nullptr || x != nullptr || rows_add != nullptr, "stream32_add_norm: nothing to add up");
    TK_CHECK_ARG(stream_out != nullptr || (w != nullptr && width <= 2048),
                 "stream32_add_norm: a row of %d without a stream to write", width);
    TK_CHECK_ARG(w == nullptr || y != nullptr, "stream32_add_norm: a norm weight without an output");
    if (rows == 0) return 0;
    if (dtype == TK_F32)
        launch_stream32<float>(stream_in, x, x_stride, rows_add, vec_add, w, eps, stream_out, y, rows, width, stream);
    else if (dtype == TK_BF16)
        launch_stream32<__nv_bfloat16>(stream_in, x, x_stride, rows_add, vec_add, w, eps, stream_out, y, rows,
                                       width, stream);
    else
        TK_CHECK_ARG(false, "stream32_add_norm: unknown dtype %d", dtype);
    TK_CHECK_LAUNCH("stream32_add_norm");
    return 0;
}

// ---------------------------------------------------------------------------------------------
// clamped gated activation: g = min(gate, limit), u = clamp(up, -limit, limit),
// out = g * sigmoid(alpha * g) * (u + shift); gu = [gate (inter) | up (inter)] per row.
// limit <= 0: no clamp.
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void glu_clamped_kernel(const T* gu, T* out, int inter, float limit, float alpha, float shift) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t t = blockIdx.x;
    const T* row = gu + t * 2 * inter;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < inter; c += gridDim.y * blockDim.x) {
        float g = to_f<T>(row[c]);
        float u = to_f<T>(row[inter + c]);
        if (limit > 0.f) {
            g = fminf(g, limit);
            u = fminf(fmaxf(u, -limit), limit);
        }
        out[t * inter + c] = from_f<T>(g / (1.0f + expf(-alpha * g)) * (u + shift));
    }
}

TK_API int tk_glu_clamped(const void* gu, void* out, int rows, int inter, float limit, float alpha, float shift,
                          int dtype, cudaStream_t stream) {
    TK_CHECK_ARG(rows >= 0 && inter > 0, "glu_clamped: bad sizes rows=%d inter=%d", rows, inter);
    if (rows == 0) return 0;
    const int threads = 256;
    const dim3 grid(rows, min(ceil_div(inter, threads), 64));
    if (dtype == TK_F32)
        tk_launch(glu_clamped_kernel<float>, grid, dim3(threads), 0, stream, (const float*)gu, (float*)out, inter, limit,
                  alpha, shift);
    else if (dtype == TK_BF16)
        tk_launch(glu_clamped_kernel<__nv_bfloat16>, grid, dim3(threads), 0, stream, (const __nv_bfloat16*)gu,
                  (__nv_bfloat16*)out, inter, limit, alpha, shift);
    else
        TK_CHECK_ARG(false, "glu_clamped: unknown dtype %d", dtype);
    TK_CHECK_LAUNCH("glu_clamped");
    return 0;
}

// ---------------------------------------------------------------------------------------------
// element-wise sigmoid gate, in place: x[t, c] = T(x[t, c] * sigmoid(g[t, c])); g's rows may be
// `ldg` elements apart (a column block of a wider projection's output)
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void sigmoid_gate_kernel(T* x, const T* g, int64_t ldg, int width) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t t = blockIdx.x;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < width; c += gridDim.y * blockDim.x) {
        const float gate = to_f<T>(g[t * ldg + c]);
        x[t * width + c] = from_f<T>(to_f<T>(x[t * width + c]) / (1.0f + expf(-gate)));
    }
}

TK_API int tk_sigmoid_gate(void* x, const void* g, int64_t ldg, int rows, int width, int dtype, cudaStream_t stream) {
    TK_CHECK_ARG(rows >= 0 && width > 0, "sigmoid_gate: bad sizes rows=%d width=%d", rows, width);
    if (rows == 0) return 0;
    const int threads = 256;
    const dim3 grid(rows, min(ceil_div(width, threads), 64));
    if (dtype == TK_F32)
        tk_launch(sigmoid_gate_kernel<float>, grid, dim3(threads), 0, stream, (float*)x, (const float*)g, ldg, width);
    else if (dtype == TK_BF16)
        tk_launch(sigmoid_gate_kernel<__nv_bfloat16>, grid, dim3(threads), 0, stream, (__nv_bfloat16*)x,
                  (const __nv_bfloat16*)g, ldg, width);
    else
        TK_CHECK_ARG(false, "sigmoid_gate: unknown dtype %d", dtype);
    TK_CHECK_LAUNCH("sigmoid_gate");
    return 0;
}
