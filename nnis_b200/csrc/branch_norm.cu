// Row-wise kernels of the arrangement whose norm stands on a sub-layer's OUTPUT:
//
//   cast_rows        x = the float32 residual rows in the operand dtype: what the
//                    sub-layers of such a block read (they read the stream itself)
//   norm_scale_add   hidden += mult * rmsnorm(branch) * w, where `branch` is what a
//                    sub-layer added up in float32; optionally also the new rows in the
//                    operand dtype, for the sub-layer that reads them next; optionally the
//                    branch rows are left zero, ready for the next sub-layer to add into
//   glu_clamp        the feed-forward activation g' sigmoid(alpha g') (u' + 1) with
//                    g' = min(g, limit), u' = clamp(u, -limit, limit)
//   tanh_rows        tanh of float32 rows, rounded once to the operand dtype
//   softcap_rows     x <- cap * tanh(x / cap), float32 in place (logits)
//   act_rows         a plain activation of float32 rows, rounded once to the operand dtype:
//                    gelu with erf, 0.5 z (1 + erf(z / sqrt 2)), or its tanh form,
//                    0.5 z (1 + tanh(sqrt(2 / pi) (z + 0.044715 z^3))), or the square of relu
//   depth_mix        keeps a block's result among the results of the blocks before it and
//                    replaces the stream by a weighted sum of them all:
//                    history[terms - 1] = hidden; hidden = sum_j w[j] history[j]
//
// Norm statistics, the scale and the sum are float32 in every dtype.
#include "async_copy.cuh"
#include "common.cuh"

namespace nnis {

template <typename T>
__global__ void cast_rows_kernel(const float* __restrict__ x, T* __restrict__ out, size_t count) {
    pdl_wait();
    pdl_launch_dependents();
    size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (i + 4 <= count) {
        store4(out + i, load4(x + i));
    } else {
        for (; i < count; ++i) out[i] = from_float<T>(x[i]);
    }
}

// a CTA of 256 threads per row
template <typename T>
__global__ void __launch_bounds__(256)
norm_scale_add_kernel(float* __restrict__ branch, const float* __restrict__ w,
                      float* __restrict__ hidden, T* __restrict__ out, int width, float eps, float mult, int clear) {
    __shared__ float red[8];
    pdl_wait();
    pdl_launch_dependents();
    const size_t row = blockIdx.x;
    float* b = branch + row * width;
    const bool by_four = (width & 3) == 0;  // rows start on 16-byte borders: four values a load
    float ss = 0.f;
    if (by_four) {
        for (int i = threadIdx.x * 4; i < width; i += 1024) {
            const float4 v = load4(b + i);
            ss = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, fmaf(v.w, v.w, ss))));
        }
    } else {
        for (int i = threadIdx.x; i < width; i += 256) ss = fmaf(b[i], b[i], ss);
    }
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float total = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) total += red[k];
    const float s = mult / sqrtf(total / (float)width + eps);
    float* h = hidden + row * width;
    if (by_four) {
        for (int i = threadIdx.x * 4; i < width; i += 1024) {
            const float4 bv = load4(b + i), wv = load4(w + i), hv = load4(h + i);
            const float4 v = make_float4(fmaf(bv.x * s, wv.x, hv.x), fmaf(bv.y * s, wv.y, hv.y),
                                         fmaf(bv.z * s, wv.z, hv.z), fmaf(bv.w * s, wv.w, hv.w));
            store4(h + i, v);
            if (out) store4(out + row * width + i, v);
            if (clear) store4(b + i, make_float4(0.f, 0.f, 0.f, 0.f));
        }
        return;
    }
    for (int i = threadIdx.x; i < width; i += 256) {
        float v = fmaf(b[i] * s, w[i], h[i]);
        h[i] = v;
        if (out) out[row * width + i] = from_float<T>(v);
        if (clear) b[i] = 0.f;
    }
}

// One to four values of a row at a time: four where rows start on 16-byte borders.
__device__ __forceinline__ void row_load(const float* p, int v, float* x) {
    if (v == 4) { const float4 t = load4(p); x[0] = t.x; x[1] = t.y; x[2] = t.z; x[3] = t.w; }
    else x[0] = p[0];
}
__device__ __forceinline__ void row_store(float* p, int v, const float* x) {
    if (v == 4) store4(p, make_float4(x[0], x[1], x[2], x[3]));
    else p[0] = x[0];
}
template <typename T>
__device__ __forceinline__ void row_store(T* p, int v, const float* x) {
    if (v == 4) store4(p, make_float4(x[0], x[1], x[2], x[3]));
    else p[0] = from_float<T>(x[0]);
}

__device__ __forceinline__ float block_sum_256(float v, float* red) {
    v = warp_sum(v);
    __syncthreads();  // (the sums of a reduction before are read)
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float total = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) total += red[k];
    return total;
}

// What closes a sub-layer of a block with a norm on either side, in one pass over the row (a CTA of 256 threads a
// row; a thread meets the same values in every loop, so only the sums need barriers):
//   hidden += rms(branch) * w, and branch is left zero;
//   with terms > 0 the new row is kept as history[terms - 1] and replaced by sum_j mix_w[j] history[j];
//   with w_next the row's RMS norm times w_next is written to `normed` in the operand dtype (the norm that reads
//   the row next: the one before the block's feed-forward, or the next block's first).
template <typename T>
__global__ void __launch_bounds__(256)
sandwich_close_kernel(float* __restrict__ branch, const float* __restrict__ w, float eps, float* __restrict__ hidden,
                      float* __restrict__ history, const float* __restrict__ mix_w, int terms, size_t plane,
                      const float* __restrict__ w_next, float eps_next, T* __restrict__ normed, int width) {
    __shared__ float red[8];
    pdl_wait();
    pdl_launch_dependents();
    const size_t row = blockIdx.x;
    float* b = branch + row * width;
    float* h = hidden + row * width;
    const int V = (width & 3) == 0 ? 4 : 1;
    float ss = 0.f;
    for (int i = threadIdx.x * V; i < width; i += 256 * V) {
        float x[4] = {0.f, 0.f, 0.f, 0.f};
        row_load(b + i, V, x);
        ss = fmaf(x[0], x[0], fmaf(x[1], x[1], fmaf(x[2], x[2], fmaf(x[3], x[3], ss))));
    }
    const float s = 1.0f / sqrtf(block_sum_256(ss, red) / (float)width + eps);
    const float zero[4] = {0.f, 0.f, 0.f, 0.f};
    float ss2 = 0.f;
    for (int i = threadIdx.x * V; i < width; i += 256 * V) {
        float bv[4], wv[4], v[4] = {0.f, 0.f, 0.f, 0.f};
        row_load(b + i, V, bv);
        row_load(w + i, V, wv);
        row_load(h + i, V, v);
        for (int e = 0; e < V; ++e) v[e] = fmaf(bv[e] * s, wv[e], v[e]);
        row_store(b + i, V, zero);
        if (terms > 0) {
            row_store(history + (size_t)(terms - 1) * plane + row * width + i, V, v);
            float sum[4] = {0.f, 0.f, 0.f, 0.f};
            for (int j = 0; j + 1 < terms; ++j) {
                float x[4];
                row_load(history + (size_t)j * plane + row * width + i, V, x);
                const float wj = mix_w[j];
                for (int e = 0; e < V; ++e) sum[e] = fmaf(wj, x[e], sum[e]);
            }
            const float wl = mix_w[terms - 1];
            for (int e = 0; e < V; ++e) v[e] = fmaf(wl, v[e], sum[e]);
        }
        row_store(h + i, V, v);
        ss2 = fmaf(v[0], v[0], fmaf(v[1], v[1], fmaf(v[2], v[2], fmaf(v[3], v[3], ss2))));
    }
    if (!w_next) return;
    const float s2 = 1.0f / sqrtf(block_sum_256(ss2, red) * (1.0f / (float)width) + eps_next);
    for (int i = threadIdx.x * V; i < width; i += 256 * V) {
        float v[4], wv[4];
        row_load(h + i, V, v);  // the thread's own values
        row_load(w_next + i, V, wv);
        for (int e = 0; e < V; ++e) v[e] = (v[e] * s2) * wv[e];
        row_store(normed + row * width + i, V, v);
    }
}

template <typename T>
__global__ void glu_clamp_kernel(const float* __restrict__ gate_up, T* __restrict__ out, size_t n_rows,
                                 int inter, float limit, float alpha) {
    pdl_wait();
    pdl_launch_dependents();
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n_rows * (size_t)inter) return;
    size_t r = idx / inter;
    int i = (int)(idx - r * inter);
    float g = fminf(gate_up[r * 2 * inter + i], limit);
    float u = fminf(fmaxf(gate_up[r * 2 * inter + inter + i], -limit), limit);
    float y = g / (1.0f + expf(-alpha * g)) * (u + 1.0f);
    out[idx] = from_float<T>(y);
}

template <typename T>
__global__ void tanh_rows_kernel(const float* __restrict__ x, T* __restrict__ out, size_t count) {
    pdl_wait();
    pdl_launch_dependents();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < count) out[i] = from_float<T>(tanhf(x[i]));
}

__global__ void softcap_rows_kernel(float* __restrict__ x, size_t count, float cap) {
    pdl_wait();
    pdl_launch_dependents();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < count) x[i] = cap * tanhf(x[i] / cap);
}

template <typename T>
__global__ void act_rows_kernel(const float* __restrict__ x, T* __restrict__ out, size_t count, int kind) {
    pdl_wait();
    pdl_launch_dependents();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= count) return;
    const float z = x[i];
    float y;
    if (kind == 0) y = 0.5f * z * (1.0f + erff(z * 0.70710678118654752f));
    else if (kind == 2) y = fmaxf(z, 0.f) * fmaxf(z, 0.f);
    else y = 0.5f * z * (1.0f + tanhf(0.79788456080286536f * (z + 0.044715f * z * z * z)));
    out[i] = from_float<T>(y);
}

// history: [terms, count] float32 (term j at j * stride); w: [terms]
__global__ void depth_mix_kernel(float* __restrict__ hidden, float* __restrict__ history,
                                 const float* __restrict__ w, size_t count, size_t stride, int terms) {
    pdl_wait();
    pdl_launch_dependents();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= count) return;
    const float x = hidden[i];
    history[(size_t)(terms - 1) * stride + i] = x;
    float sum = 0.f;
    for (int j = 0; j + 1 < terms; ++j) sum = fmaf(w[j], history[(size_t)j * stride + i], sum);
    hidden[i] = fmaf(w[terms - 1], x, sum);
}

}  // namespace nnis

using namespace nnis;

// kind 0: gelu (erf); 1: gelu (tanh form)
NNIS_API int nnis_act_rows(const float* x, void* out, int out_dtype, long long count, int kind,
                           cudaStream_t stream) {
    if (count <= 0 || !x || !out || kind < 0 || kind > 2) return NNIS_ERR_ARGUMENT;
    unsigned blocks = (unsigned)((count + 255) / 256);
    cudaError_t e;
    if (out_dtype == NNIS_DTYPE_F32)
        e = launch_dependent(act_rows_kernel<float>, blocks, 256, 0, stream, x, (float*)out, (size_t)count, kind);
    else if (out_dtype == NNIS_DTYPE_BF16)
        e = launch_dependent(act_rows_kernel<bf16>, blocks, 256, 0, stream, x, (bf16*)out, (size_t)count, kind);
    else
        return NNIS_ERR_UNSUPPORTED;
    return e == cudaSuccess ? NNIS_OK : (int)e;
}

NNIS_API int nnis_depth_mix(float* hidden, float* history, const float* w, long long count, long long stride,
                            int terms, cudaStream_t stream) {
    if (count <= 0 || stride < count || terms <= 0 || !hidden || !history || !w) return NNIS_ERR_ARGUMENT;
    unsigned blocks = (unsigned)((count + 255) / 256);
    cudaError_t e = launch_dependent(depth_mix_kernel, blocks, 256, 0, stream, hidden, history, w, (size_t)count,
                                     (size_t)stride, terms);
    return e == cudaSuccess ? NNIS_OK : (int)e;
}

NNIS_API int nnis_cast_rows(const float* x, void* out, int out_dtype, long long count, cudaStream_t stream) {
    if (count <= 0 || !x || !out) return NNIS_ERR_ARGUMENT;
    unsigned blocks = (unsigned)(((count + 3) / 4 + 255) / 256);
    cudaError_t e;
    if (out_dtype == NNIS_DTYPE_F32)
        e = launch_dependent(cast_rows_kernel<float>, blocks, 256, 0, stream, x, (float*)out, (size_t)count);
    else if (out_dtype == NNIS_DTYPE_BF16)
        e = launch_dependent(cast_rows_kernel<bf16>, blocks, 256, 0, stream, x, (bf16*)out, (size_t)count);
    else
        return NNIS_ERR_UNSUPPORTED;
    return e == cudaSuccess ? NNIS_OK : (int)e;
}

// out may be null (no copy in the operand dtype is wanted); clear: the branch rows are zero afterwards
NNIS_API int nnis_norm_scale_add(float* branch, const float* w, float* hidden, void* out, int out_dtype,
                                 int n_rows, int width, float eps, float mult, int clear, cudaStream_t stream) {
    if (n_rows <= 0 || width <= 0 || !(eps > 0.f) || !branch || !w || !hidden) return NNIS_ERR_ARGUMENT;
    cudaError_t e;
    if (out_dtype == NNIS_DTYPE_F32)
        e = launch_dependent(norm_scale_add_kernel<float>, (unsigned)n_rows, 256, 0, stream, branch, w, hidden,
                             (float*)out, width, eps, mult, clear);
    else if (out_dtype == NNIS_DTYPE_BF16)
        e = launch_dependent(norm_scale_add_kernel<bf16>, (unsigned)n_rows, 256, 0, stream, branch, w, hidden,
                             (bf16*)out, width, eps, mult, clear);
    else
        return NNIS_ERR_UNSUPPORTED;
    return e == cudaSuccess ? NNIS_OK : (int)e;
}

// history [at least terms, n_rows, width] and mix_w [terms] with terms > 0, else unused; w_next and normed
// (operand dtype) together or neither
NNIS_API int nnis_sandwich_close(float* branch, const float* w, float eps, float* hidden, float* history,
                                 const float* mix_w, int terms, const float* w_next, float eps_next, void* normed,
                                 int out_dtype, int n_rows, int width, cudaStream_t stream) {
    if (n_rows <= 0 || width <= 0 || !(eps > 0.f) || !branch || !w || !hidden || terms < 0 ||
        (terms > 0 && (!history || !mix_w)) || (!w_next != !normed) || (w_next && !(eps_next > 0.f)))
        return NNIS_ERR_ARGUMENT;
    const size_t plane = (size_t)n_rows * width;
    cudaError_t e;
    if (out_dtype == NNIS_DTYPE_F32)
        e = launch_dependent(sandwich_close_kernel<float>, (unsigned)n_rows, 256, 0, stream, branch, w, eps, hidden,
                             history, mix_w, terms, plane, w_next, eps_next, (float*)normed, width);
    else if (out_dtype == NNIS_DTYPE_BF16)
        e = launch_dependent(sandwich_close_kernel<bf16>, (unsigned)n_rows, 256, 0, stream, branch, w, eps, hidden,
                             history, mix_w, terms, plane, w_next, eps_next, (bf16*)normed, width);
    else
        return NNIS_ERR_UNSUPPORTED;
    return e == cudaSuccess ? NNIS_OK : (int)e;
}

NNIS_API int nnis_glu_clamp(const float* gate_up, void* out, int out_dtype, long long n_rows, int inter,
                            float limit, float alpha, cudaStream_t stream) {
    if (n_rows <= 0 || inter <= 0 || !(limit > 0.f)) return NNIS_ERR_ARGUMENT;
    size_t total = (size_t)n_rows * inter;
    unsigned blocks = (unsigned)((total + 255) / 256);
    cudaError_t e;
    if (out_dtype == NNIS_DTYPE_F32)
        e = launch_dependent(glu_clamp_kernel<float>, blocks, 256, 0, stream, gate_up, (float*)out, (size_t)n_rows,
                             inter, limit, alpha);
    else if (out_dtype == NNIS_DTYPE_BF16)
        e = launch_dependent(glu_clamp_kernel<bf16>, blocks, 256, 0, stream, gate_up, (bf16*)out, (size_t)n_rows,
                             inter, limit, alpha);
    else
        return NNIS_ERR_UNSUPPORTED;
    return e == cudaSuccess ? NNIS_OK : (int)e;
}

NNIS_API int nnis_tanh_rows(const float* x, void* out, int out_dtype, long long count, cudaStream_t stream) {
    if (count <= 0 || !x || !out) return NNIS_ERR_ARGUMENT;
    unsigned blocks = (unsigned)((count + 255) / 256);
    cudaError_t e;
    if (out_dtype == NNIS_DTYPE_F32)
        e = launch_dependent(tanh_rows_kernel<float>, blocks, 256, 0, stream, x, (float*)out, (size_t)count);
    else if (out_dtype == NNIS_DTYPE_BF16)
        e = launch_dependent(tanh_rows_kernel<bf16>, blocks, 256, 0, stream, x, (bf16*)out, (size_t)count);
    else
        return NNIS_ERR_UNSUPPORTED;
    return e == cudaSuccess ? NNIS_OK : (int)e;
}

NNIS_API int nnis_softcap_rows(float* x, long long count, float cap, cudaStream_t stream) {
    if (count <= 0 || !x || !(cap > 0.f)) return NNIS_ERR_ARGUMENT;
    unsigned blocks = (unsigned)((count + 255) / 256);
    cudaError_t e = launch_dependent(softcap_rows_kernel, blocks, 256, 0, stream, x, (size_t)count, cap);
    return e == cudaSuccess ? NNIS_OK : (int)e;
}
