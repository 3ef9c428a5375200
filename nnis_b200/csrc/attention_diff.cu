// Differential attention over the paged cache: every head has TWO attention maps over the same
// values, and its output is their difference, normed.
//
// A query head holds [q1 | q2] (2 dk values), a key head [k1 | k2] (a cache row of 2 dk values);
// map c is softmax(scale * q_c . k_c) over the keys the mask lets through (causal; with window > 0
// only j > p - window).  With a1, a2 the two maps' weighted sums of the SAME value rows:
//
//     o = a1 - lambda * a2;   out = o / sqrt(mean(o^2) + eps) * post * gate
//
// over the head's dv values (lambda, post: numbers of the layer; gate: float32 [n, heads * dv] or
// null).  Scores, softmax, the difference and its norm are float32 in every dtype.
//
//   attn_diff        one warp per (query token, G query heads of one key/value head): a lane takes a
//                    key, computes its 2 G scores from one fetched key row, and one fetched value row
//                    feeds 2 G accumulators.  The key range may be cut into slices that leave partial
//                    records [m1, l1, m2, l2, acc1 (dv), acc2 (dv)].
//   attn_diff_merge  the slices of a (token, head) put together in ascending order, then the
//                    difference, the norm and the gate.
//
// Serves prompts and single tokens, float32 and bfloat16 storage.  A row whose position is -1
// (padding) is skipped.
#include <float.h>

#include "async_copy.cuh"
#include "common.cuh"

namespace nnis {

template <typename T, int R, int G>
__global__ void __launch_bounds__(128)
attn_diff_kernel(const T* __restrict__ q, const T* __restrict__ k_cache, const T* __restrict__ v_cache,
                 const int* __restrict__ token_pos, const int* __restrict__ token_seq,
                 const int* __restrict__ page_table, int table_cols, const float* __restrict__ gate,
                 T* __restrict__ out, float* __restrict__ partial, int n_tokens, int nq, int nkv, int dk, int dv,
                 int page_size, int window, float scale, float lambda, float post, float eps, int n_splits) {
    extern __shared__ __align__(16) float q_smem[];  // [4 warps][G][2 dk]
    pdl_wait();
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int n = blockIdx.x * 4 + warp;
    if (n >= n_tokens) return;
    const int h0 = blockIdx.y * G, split = blockIdx.z;
    const int hk = h0 / (nq / nkv);
    const int pos = token_pos[n];
    const int dk2 = 2 * dk;
    constexpr int VB = R <= 2 ? 8 : 4;  // value rows in flight a lane (32 / VB loads of R values each)
    float* qs = q_smem + (size_t)warp * G * dk2;

    float m[G][2], l[G][2], acc[G][2][R];
#pragma unroll
    for (int g = 0; g < G; ++g)
#pragma unroll
        for (int c = 0; c < 2; ++c) {
            m[g][c] = -FLT_MAX;
            l[g][c] = 0.f;
#pragma unroll
            for (int r = 0; r < R; ++r) acc[g][c][r] = 0.f;
        }
    if (pos < 0) {
        if (n_splits == 1) return;
    } else {
        const T* qrow = q + ((size_t)n * nq + h0) * dk2;  // the group's heads are neighbours
        for (int i = lane; i < G * dk2; i += 32) qs[i] = to_float(qrow[i]);
        __syncwarp();
        const int lo = window > 0 ? max(0, pos - window + 1) : 0;
        const int hi = pos + 1;
        int per = (hi - lo + n_splits - 1) / n_splits;
        per = (per + 31) & ~31;
        const int start = lo + split * per;
        const int end = min(hi, start + per);
        const int* table = page_table + (size_t)token_seq[n] * table_cols;
        const bool by_four = (dk & 3) == 0;
        for (int t0 = start; t0 < end; t0 += 32) {
            const int t = t0 + lane;
            const bool valid = t < end;
            int row_index = 0;
            float s[G][2];
#pragma unroll
            for (int g = 0; g < G; ++g) s[g][0] = s[g][1] = 0.f;
            if (valid) {
                const int page = table[t / page_size];
                row_index = (page * nkv + hk) * page_size + (t % page_size);
                const T* krow = k_cache + (size_t)row_index * dk2;
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    if (by_four) {
#pragma unroll 8
                        for (int i = 0; i < dk; i += 4) {
                            const float4 kv = load4(krow + c * dk + i);
#pragma unroll
                            for (int g = 0; g < G; ++g) {
                                const float4 qv = *reinterpret_cast<const float4*>(qs + g * dk2 + c * dk + i);
                                s[g][c] = fmaf(qv.x, kv.x, s[g][c]);
                                s[g][c] = fmaf(qv.y, kv.y, s[g][c]);
                                s[g][c] = fmaf(qv.z, kv.z, s[g][c]);
                                s[g][c] = fmaf(qv.w, kv.w, s[g][c]);
                            }
                        }
                    } else {
                        for (int i = 0; i < dk; ++i) {
                            const float kv = to_float(krow[c * dk + i]);
#pragma unroll
                            for (int g = 0; g < G; ++g) s[g][c] = fmaf(qs[g * dk2 + c * dk + i], kv, s[g][c]);
                        }
                    }
                }
            }
            float p[G][2];
#pragma unroll
            for (int g = 0; g < G; ++g)
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    const float sv = valid ? s[g][c] * scale : -FLT_MAX;
                    const float m_new = fmaxf(m[g][c], warp_max(sv));
                    p[g][c] = valid ? expf(sv - m_new) : 0.f;
                    const float alpha = l[g][c] == 0.f ? 0.f : expf(m[g][c] - m_new);
                    l[g][c] = l[g][c] * alpha + warp_sum(p[g][c]);
                    m[g][c] = m_new;
#pragma unroll
                    for (int r = 0; r < R; ++r) acc[g][c][r] *= alpha;
                }
            // the value rows of VB keys are asked for together, then added: a row's load waits for none
            // of the others (keys past the end have weight zero and row 0, which is there to be read)
            const int count = min(32, end - t0);
            for (int j0 = 0; j0 < count; j0 += VB) {
                float vr[VB][R];
#pragma unroll
                for (int u = 0; u < VB; ++u) {
                    const int rj = __shfl_sync(0xffffffffu, row_index, j0 + u);
                    const T* vrow = v_cache + (size_t)rj * dv;
#pragma unroll
                    for (int r = 0; r < R; ++r) {
                        const int i = lane + 32 * r;
                        vr[u][r] = i < dv ? to_float(vrow[i]) : 0.f;
                    }
                }
#pragma unroll
                for (int u = 0; u < VB; ++u)
#pragma unroll
                    for (int g = 0; g < G; ++g)
#pragma unroll
                        for (int c = 0; c < 2; ++c) {
                            const float pj = __shfl_sync(0xffffffffu, p[g][c], j0 + u);
#pragma unroll
                            for (int r = 0; r < R; ++r) acc[g][c][r] = fmaf(pj, vr[u][r], acc[g][c][r]);
                        }
            }
        }
    }
#pragma unroll
    for (int g = 0; g < G; ++g) {
        const int hq = h0 + g;
        if (n_splits == 1) {
            const float inv1 = l[g][0] > 0.f ? 1.0f / l[g][0] : 0.f;
            const float inv2 = l[g][1] > 0.f ? 1.0f / l[g][1] : 0.f;
            float o[R], ss = 0.f;
#pragma unroll
            for (int r = 0; r < R; ++r) {
                o[r] = acc[g][0][r] * inv1 - lambda * (acc[g][1][r] * inv2);  // (lanes beyond dv hold zeros)
                ss = fmaf(o[r], o[r], ss);
            }
            ss = warp_sum(ss);
            const float unit = post / sqrtf(ss / (float)dv + eps);
            const float* ge = gate ? gate + ((size_t)n * nq + hq) * dv : nullptr;
            T* dst = out + ((size_t)n * nq + hq) * dv;
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const int i = lane + 32 * r;
                if (i < dv) dst[i] = from_float<T>(o[r] * unit * (ge ? ge[i] : 1.0f));
            }
        } else {
            float* rec = partial + (((size_t)n * nq + hq) * n_splits + split) * (size_t)(2 * dv + 4);
            if (lane == 0) {
                rec[0] = m[g][0];
                rec[1] = l[g][0];
                rec[2] = m[g][1];
                rec[3] = l[g][1];
            }
#pragma unroll
            for (int c = 0; c < 2; ++c)
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    const int i = lane + 32 * r;
                    if (i < dv) rec[4 + c * dv + i] = acc[g][c][r];
                }
        }
    }
}

// A CTA of 128 threads per (token, head), at most 64 slices, dv <= 256.
template <typename T>
__global__ void __launch_bounds__(128)
attn_diff_merge_kernel(const float* __restrict__ partial, const int* __restrict__ token_pos,
                       const float* __restrict__ gate, T* __restrict__ out, int nq, int dv, int n_splits,
                       float lambda, float post, float eps) {
    __shared__ float share[2][64];
    __shared__ float red[4];
    pdl_wait();
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const size_t row = blockIdx.x;
    if (token_pos[row / nq] < 0) return;
    const size_t rec_size = 2 * (size_t)dv + 4;
    const float* rec = partial + row * n_splits * rec_size;
    if (warp < 2) {  // warp c works out the weights exp(m_s - m) / l of map c's slices
        float ms[2], ls[2];
        float mx = -FLT_MAX;
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            const int s = lane + 32 * k;
            ms[k] = s < n_splits ? rec[(size_t)s * rec_size + 2 * warp] : 0.f;
            ls[k] = s < n_splits ? rec[(size_t)s * rec_size + 2 * warp + 1] : 0.f;
            if (ls[k] > 0.f) mx = fmaxf(mx, ms[k]);
        }
        mx = warp_max(mx);
        float l = 0.f;
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            ms[k] = ls[k] > 0.f ? expf(ms[k] - mx) : 0.f;
            l += ls[k] * ms[k];
        }
        l = warp_sum(l);
        const float inv = l > 0.f ? 1.0f / l : 0.f;
        share[warp][lane] = ms[0] * inv;
        share[warp][lane + 32] = ms[1] * inv;
    }
    __syncthreads();
    float o[2], ss = 0.f;
#pragma unroll
    for (int k = 0; k < 2; ++k) {
        const int i = threadIdx.x + 128 * k;
        o[k] = 0.f;
        if (i < dv) {
            float a1 = 0.f, a2 = 0.f;
            for (int s = 0; s < n_splits; ++s) {
                const float w1 = share[0][s], w2 = share[1][s];
                if (w1 > 0.f) a1 = fmaf(w1, rec[(size_t)s * rec_size + 4 + i], a1);
                if (w2 > 0.f) a2 = fmaf(w2, rec[(size_t)s * rec_size + 4 + dv + i], a2);
            }
            o[k] = a1 - lambda * a2;
            ss = fmaf(o[k], o[k], ss);
        }
    }
    ss = warp_sum(ss);
    if (lane == 0) red[warp] = ss;
    __syncthreads();
    ss = red[0] + red[1] + red[2] + red[3];
    const float unit = post / sqrtf(ss / (float)dv + eps);
#pragma unroll
    for (int k = 0; k < 2; ++k) {
        const int i = threadIdx.x + 128 * k;
        if (i < dv) out[row * dv + i] = from_float<T>(o[k] * unit * (gate ? gate[row * dv + i] : 1.0f));
    }
}

template <typename T, int G>
static cudaError_t launch_diff_r(dim3 grid, size_t smem, cudaStream_t stream, const void* q, const void* k_cache,
                                 const void* v_cache, const int* token_pos, const int* token_seq,
                                 const int* page_table, int table_cols, const float* gate, void* out, float* partial,
                                 int n_tokens, int nq, int nkv, int dk, int dv, int page_size, int window,
                                 float scale, float lambda, float post, float eps, int n_splits) {
#define NNIS_DIFF_CASE(R) \
    return launch_dependent(attn_diff_kernel<T, R, G>, grid, 128, smem, stream, (const T*)q, (const T*)k_cache, \
                            (const T*)v_cache, token_pos, token_seq, page_table, table_cols, gate, (T*)out, partial, \
                            n_tokens, nq, nkv, dk, dv, page_size, window, scale, lambda, post, eps, n_splits)
    if (dv <= 32) NNIS_DIFF_CASE(1);
    if (dv <= 64) NNIS_DIFF_CASE(2);
    if (dv <= 128) NNIS_DIFF_CASE(4);
    NNIS_DIFF_CASE(8);
#undef NNIS_DIFF_CASE
}

template <typename T>
static int launch_attn_diff(const void* q, const void* k_cache, const void* v_cache, const int* token_pos,
                            const int* token_seq, const int* page_table, int table_cols, const float* gate,
                            void* out, float* partial, int n_tokens, int nq, int nkv, int dk, int dv, int page_size,
                            int window, float scale, float lambda, float post, float eps, int n_splits,
                            cudaStream_t stream) {
    const int group = nq / nkv;
    // as many query heads of a key/value head in one warp as divide the group and fit registers and
    // shared memory
    int G = (group % 4 == 0 && dv <= 128) ? 4 : (group % 2 == 0 ? 2 : 1);
    while (G > 1 && 4 * (size_t)G * 2 * dk * sizeof(float) > 48 * 1024) G >>= 1;
    const size_t smem = 4 * (size_t)G * 2 * dk * sizeof(float);
    if (smem > 48 * 1024) return NNIS_ERR_UNSUPPORTED;
    dim3 grid((n_tokens + 3) / 4, nq / G, n_splits);
    cudaError_t e;
    if (G == 4)
        e = launch_diff_r<T, 4>(grid, smem, stream, q, k_cache, v_cache, token_pos, token_seq, page_table, table_cols,
                                gate, out, partial, n_tokens, nq, nkv, dk, dv, page_size, window, scale, lambda, post,
                                eps, n_splits);
    else if (G == 2)
        e = launch_diff_r<T, 2>(grid, smem, stream, q, k_cache, v_cache, token_pos, token_seq, page_table, table_cols,
                                gate, out, partial, n_tokens, nq, nkv, dk, dv, page_size, window, scale, lambda, post,
                                eps, n_splits);
    else
        e = launch_diff_r<T, 1>(grid, smem, stream, q, k_cache, v_cache, token_pos, token_seq, page_table, table_cols,
                                gate, out, partial, n_tokens, nq, nkv, dk, dv, page_size, window, scale, lambda, post,
                                eps, n_splits);
    if (e != cudaSuccess) return (int)e;
    if (n_splits > 1) {
        const size_t rows = (size_t)n_tokens * nq;
        e = launch_dependent(attn_diff_merge_kernel<T>, (unsigned)rows, 128, 0, stream, (const float*)partial,
                             token_pos, gate, (T*)out, nq, dv, n_splits, lambda, post, eps);
    }
    return e == cudaSuccess ? NNIS_OK : (int)e;
}

}  // namespace nnis

using namespace nnis;

// q: [n, nq * 2 dk]; caches [pages, nkv, page, 2 dk] and [pages, nkv, page, dv]; gate: float32
// [n, nq * dv] or null; out [n, nq * dv]; partial: n * nq * n_splits * (2 dv + 4) floats when
// n_splits > 1.  dk: the size of ONE map's query and key.
NNIS_API int nnis_attention_diff(const void* q, const void* k_cache, const void* v_cache, const int* token_pos,
                                 const int* token_seq, const int* page_table, int table_cols, const float* gate,
                                 void* out, float* partial, int n_tokens, int nq, int nkv, int dk, int dv,
                                 int page_size, int window, float scale, float lambda, float post, float eps,
                                 int n_splits, int dtype, cudaStream_t stream) {
    if (n_tokens <= 0 || nq <= 0 || nkv <= 0 || nq % nkv || page_size <= 0 || table_cols <= 0 || n_splits <= 0 ||
        window < 0 || !(eps > 0.f) || !q || !k_cache || !v_cache || !token_pos || !token_seq || !page_table || !out)
        return NNIS_ERR_ARGUMENT;
    if (dk <= 0 || dv <= 0 || dk > 512 || dv > 256) return NNIS_ERR_UNSUPPORTED;
    if (nq > 65535 || n_splits > 64) return NNIS_ERR_UNSUPPORTED;
    if (n_splits > 1 && !partial) return NNIS_ERR_ARGUMENT;
    if (dtype == NNIS_DTYPE_F32)
        return launch_attn_diff<float>(q, k_cache, v_cache, token_pos, token_seq, page_table, table_cols, gate, out,
                                       partial, n_tokens, nq, nkv, dk, dv, page_size, window, scale, lambda, post,
                                       eps, n_splits, stream);
    if (dtype == NNIS_DTYPE_BF16)
        return launch_attn_diff<bf16>(q, k_cache, v_cache, token_pos, token_seq, page_table, table_cols, gate, out,
                                      partial, n_tokens, nq, nkv, dk, dv, page_size, window, scale, lambda, post,
                                      eps, n_splits, stream);
    return NNIS_ERR_UNSUPPORTED;
}
