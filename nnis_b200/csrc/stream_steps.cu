// Row-wise steps on the float32 residual stream that are no part of a sub-layer.
//
//   embed_pair     hidden[n] = table[token] * scale + pair[row]: the token's embedding times a
//                  number, plus a row of a second table chosen by a hash of (the token before,
//                  the token): (prev * mul_prev + token * mul_cur) mod buckets, and row `buckets`
//                  for a sequence's first token.  The token before the first row of a step's
//                  portion is the sequence's state (`last_token[slot]`); the CTA of that row
//                  reads it and then leaves the portion's last token there, so no other CTA
//                  touches the slot's entry.
//   rmsnorm_pair   two RMS norms of the same rows with weights of their own: one pass, one
//                  statistic, two outputs (the arrangement whose two branches read norms of
//                  the same stream).
//   stream_enter   hidden[n] += kept[n] + row: what a pass through a run of layers adds to the
//                  stream before its first layer (both terms optional).
//   scale_rows     x *= s on float32 rows (logits).
//
// A row whose position is -1 (padding) gets zeros from embed_pair and is left alone by no
// other kernel here: its values reach no result.
#include "async_copy.cuh"
#include "common.cuh"

namespace nnis {

template <typename T>
__global__ void __launch_bounds__(256)
embed_pair_kernel(const T* __restrict__ table, const T* __restrict__ pair, const int* __restrict__ tokens,
                  const int* __restrict__ token_pos, const int* __restrict__ token_seq,
                  const int* __restrict__ seq_slots, const int* __restrict__ seq_count,
                  int* __restrict__ last_token, float* __restrict__ hidden, int width, int vocab, int buckets,
                  long long mul_prev, long long mul_cur, float scale, int* __restrict__ status) {
    __shared__ int pair_row_s;
    const int n = blockIdx.x;
    const int pos = token_pos[n];
    float* out = hidden + (size_t)n * width;
    if (pos < 0) {
        for (int i = threadIdx.x; i < width; i += blockDim.x) out[i] = 0.f;
        return;
    }
    int token = tokens[n];
    const bool bad = token < 0 || token >= vocab;
    if (bad) {
        if (threadIdx.x == 0) atomicExch(status, 1);
        token = 0;
    }
    if (threadIdx.x == 0) {
        const int seq = token_seq[n];
        // the first row that this step brings of its sequence
        const bool first = n == 0 || token_seq[n - 1] != seq || token_pos[n - 1] < 0;
        int row = buckets;
        if (pair) {
            if (pos > 0) {
                const long long prev = first ? last_token[seq_slots[seq]] : tokens[n - 1];
                long long h = (prev * mul_prev + (long long)token * mul_cur) % buckets;
                row = (int)(h < 0 ? h + buckets : h);
            }
            if (first) last_token[seq_slots[seq]] = tokens[n + (seq_count ? seq_count[seq] : 1) - 1];
        }
        pair_row_s = row;
    }
    __syncthreads();
    const T* row = table + (size_t)token * width;
    const T* extra = pair ? pair + (size_t)pair_row_s * width : nullptr;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        float v = to_float(row[i]) * scale;
        if (extra) v += to_float(extra[i]);
        out[i] = bad ? 0.f : v;
    }
}

// a CTA per row
template <typename T>
__global__ void __launch_bounds__(256)
rmsnorm_pair_kernel(const float* __restrict__ x, const float* __restrict__ w1, const float* __restrict__ w2,
                    T* __restrict__ y1, T* __restrict__ y2, int width, float eps) {
    __shared__ float partial[8];
    __shared__ float scale_s;
    pdl_wait();
    pdl_launch_dependents();
    const int r = blockIdx.x;
    const float* in = x + (size_t)r * width;
    float ss = 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) ss = fmaf(in[i], in[i], ss);
    ss = warp_sum(ss);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    if (lane == 0) partial[warp] = ss;
    __syncthreads();
    if (warp == 0) {
        float v = lane < n_warps ? partial[lane] : 0.f;
        v = warp_sum(v);
        if (lane == 0) scale_s = 1.0f / sqrtf(v * (1.0f / (float)width) + eps);
    }
    __syncthreads();
    const float s = scale_s;
    T* o1 = y1 + (size_t)r * width;
    T* o2 = y2 + (size_t)r * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float v = in[i] * s;
        o1[i] = from_float<T>(v * w1[i]);
        o2[i] = from_float<T>(v * w2[i]);
    }
}

// a warp per row, the row in registers between the sum and the two outputs (width % 4 == 0, <= 1,024)
template <typename T>
__global__ void __launch_bounds__(256)
rmsnorm_pair_rows_kernel(const float* __restrict__ x, const float* __restrict__ w1, const float* __restrict__ w2,
                         T* __restrict__ y1, T* __restrict__ y2, int n_rows, int width, float eps) {
    const int lane = threadIdx.x & 31, r = blockIdx.x * 8 + (threadIdx.x >> 5);
    const int n4 = width >> 2;
    pdl_wait();
    pdl_launch_dependents();
    if (r >= n_rows) return;
    const float4* in = reinterpret_cast<const float4*>(x + (size_t)r * width);
    float4 v[8];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const int c = lane + 32 * j;
        v[j] = c < n4 ? in[c] : make_float4(0.f, 0.f, 0.f, 0.f);
        ss = fmaf(v[j].x, v[j].x, ss);
        ss = fmaf(v[j].y, v[j].y, ss);
        ss = fmaf(v[j].z, v[j].z, ss);
        ss = fmaf(v[j].w, v[j].w, ss);
    }
    ss = warp_sum(ss);
    const float s = 1.0f / sqrtf(ss * (1.0f / (float)width) + eps);
    const float4* g1 = reinterpret_cast<const float4*>(w1);
    const float4* g2 = reinterpret_cast<const float4*>(w2);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const int c = lane + 32 * j;
        if (c < n4) {
            const float4 a = g1[c], b = g2[c];
            const float4 u = make_float4(v[j].x * s, v[j].y * s, v[j].z * s, v[j].w * s);
            store4(y1 + (size_t)r * width + c * 4, make_float4(u.x * a.x, u.y * a.y, u.z * a.z, u.w * a.w));
            store4(y2 + (size_t)r * width + c * 4, make_float4(u.x * b.x, u.y * b.y, u.z * b.z, u.w * b.w));
        }
    }
}

__global__ void stream_enter_kernel(float* __restrict__ hidden, const float* __restrict__ kept,
                                    const float* __restrict__ row, size_t count, int width) {
    pdl_wait();
    pdl_launch_dependents();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= count) return;
    float v = hidden[i];
    if (kept) v += kept[i];
    if (row) v += row[i % width];
    hidden[i] = v;
}

__global__ void scale_rows_kernel(float* __restrict__ x, size_t count, float s) {
    pdl_wait();
    pdl_launch_dependents();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < count) x[i] *= s;
}

}  // namespace nnis

using namespace nnis;

// table [vocab, width], pair [buckets + 1, width] or null (then no state is read or written);
// seq_count: int32 per sequence of the step, or null when every sequence brings one token;
// last_token: int32 [slots]
NNIS_API int nnis_embed_pair(const void* table, const void* pair, int dtype, const int* tokens,
                             const int* token_pos, const int* token_seq, const int* seq_slots,
                             const int* seq_count, int* last_token, float* hidden, int n_tokens, int width,
                             int vocab, int buckets, long long mul_prev, long long mul_cur, float scale,
                             int* status, cudaStream_t stream) {
    if (n_tokens <= 0 || width <= 0 || vocab <= 0 || !table || !tokens || !token_pos || !hidden || !status)
        return NNIS_ERR_ARGUMENT;
    if (pair && (buckets <= 0 || !token_seq || !seq_slots || !last_token)) return NNIS_ERR_ARGUMENT;
    const int threads = width >= 256 ? 256 : 64;
    if (dtype == NNIS_DTYPE_F32)
        embed_pair_kernel<float><<<n_tokens, threads, 0, stream>>>(
            (const float*)table, (const float*)pair, tokens, token_pos, token_seq, seq_slots, seq_count, last_token,
            hidden, width, vocab, buckets, mul_prev, mul_cur, scale, status);
    else if (dtype == NNIS_DTYPE_BF16)
        embed_pair_kernel<bf16><<<n_tokens, threads, 0, stream>>>(
            (const bf16*)table, (const bf16*)pair, tokens, token_pos, token_seq, seq_slots, seq_count, last_token,
            hidden, width, vocab, buckets, mul_prev, mul_cur, scale, status);
    else
        return NNIS_ERR_UNSUPPORTED;
    NNIS_RETURN_LAUNCH();
}

NNIS_API int nnis_rmsnorm_pair(const float* x, const float* w1, const float* w2, void* y1, void* y2, int out_dtype,
                               int n_rows, int width, float eps, cudaStream_t stream) {
    if (n_rows <= 0 || width <= 0 || !(eps > 0.f) || !x || !w1 || !w2 || !y1 || !y2) return NNIS_ERR_ARGUMENT;
    const bool by_rows = n_rows >= 64 && width % 4 == 0 && width <= 1024 &&
                         ((uintptr_t)x | (uintptr_t)w1 | (uintptr_t)w2 | (uintptr_t)y1 | (uintptr_t)y2) % 16 == 0;
    const unsigned grid = by_rows ? (n_rows + 7) / 8 : n_rows;
    const unsigned block = by_rows ? 256 : (width >= 1024 ? 256 : (width >= 256 ? 128 : 32));
    cudaError_t e;
    if (out_dtype == NNIS_DTYPE_F32)
        e = by_rows ? launch_dependent(rmsnorm_pair_rows_kernel<float>, grid, block, 0, stream, x, w1, w2, (float*)y1,
                                       (float*)y2, n_rows, width, eps)
                    : launch_dependent(rmsnorm_pair_kernel<float>, grid, block, 0, stream, x, w1, w2, (float*)y1,
                                       (float*)y2, width, eps);
    else if (out_dtype == NNIS_DTYPE_BF16)
        e = by_rows ? launch_dependent(rmsnorm_pair_rows_kernel<bf16>, grid, block, 0, stream, x, w1, w2, (bf16*)y1,
                                       (bf16*)y2, n_rows, width, eps)
                    : launch_dependent(rmsnorm_pair_kernel<bf16>, grid, block, 0, stream, x, w1, w2, (bf16*)y1,
                                       (bf16*)y2, width, eps);
    else
        return NNIS_ERR_UNSUPPORTED;
    return e == cudaSuccess ? NNIS_OK : (int)e;
}

// hidden float32 [count]; kept float32 [count] or null; row float32 [width] or null
NNIS_API int nnis_stream_enter(float* hidden, const float* kept, const float* row, long long count, int width,
                               cudaStream_t stream) {
    if (count <= 0 || width <= 0 || !hidden || (!kept && !row)) return NNIS_ERR_ARGUMENT;
    const unsigned blocks = (unsigned)((count + 255) / 256);
    cudaError_t e = launch_dependent(stream_enter_kernel, blocks, 256, 0, stream, hidden, kept, row, (size_t)count,
                                     width);
    return e == cudaSuccess ? NNIS_OK : (int)e;
}

NNIS_API int nnis_scale_rows(float* x, long long count, float s, cudaStream_t stream) {
    if (count <= 0 || !x) return NNIS_ERR_ARGUMENT;
    const unsigned blocks = (unsigned)((count + 255) / 256);
    cudaError_t e = launch_dependent(scale_rows_kernel, blocks, 256, 0, stream, x, (size_t)count, s);
    return e == cudaSuccess ? NNIS_OK : (int)e;
}
