// Attention with a soft cap on its scores, a sink in the softmax's denominator, a chunked
// or windowed causal mask, key and value heads of different sizes and a gate per head, over
// the paged cache; and the row-wise step in front of it.
//
//   qkv_prep        from the projection's float32 rows [q (H dk) | k (G dk) | v (G dv) | gate (H)]:
//                   RMS norm of q and of k over the WHOLE projection (all heads at once, one
//                   weight per column), rotation of neighbouring pairs (2i, 2i + 1) of the first
//                   `rot` values of every head by position * freq[i], q to a packed buffer, k and
//                   v into the cache row of the token, sigmoid of the gate's logits.  Every part
//                   is optional (no norm weights, rot 0, no k/v in the rows, no gate).
//   qkv_prep_heads  the same step with everything per head: rotation of either pairing (neighbours, or
//                   value i with value i + rot / 2), then optionally an RMS norm of every q and k head
//                   by itself (no weight, after the rotation), optionally a number per query head that
//                   multiplies its q (a temperature of the scores), and `gate_cols` gate logits a token
//                   (one per head, or one per output value).  A head may hold `maps` vectors of equal
//                   size side by side (the queries and keys of several attention maps over one set of
//                   values); each is turned by itself over its own first `rot` values.  `magnitude`
//                   multiplies every cosine and sine (1: a pure rotation).
//   attn_sink       one warp per (query token, query head) walks the visible keys 32 at a time with
//                   an online softmax in float32: score = cap * tanh(scale * q.k / cap) (cap 0: none);
//                   a query at position p sees keys j <= p with j >= p - window + 1 (window > 0) and
//                   floor(j / chunk) == floor(p / chunk) (chunk > 0, chunks counted from position 0 of
//                   the sequence); the denominator also holds exp(sink[head]), which has no key and
//                   no value; the output is multiplied by gate[token, head] (or, with `gate_elems` = dv, value by value
//                   by gate[token, head, :]).  The key range may be
//                   cut into slices whose partial records a second kernel merges in order (the sink
//                   counts in the first slice).
//   attn_sink_group the same where 2, 3, 4, 6 or 8 query heads share a key/value head: one warp per
//                   (query token, key/value head) holds all its query heads, so a key's and a value's
//                   row is fetched once for the group instead of once a head.
//
// Serves prompts and single tokens, float32 and bfloat16 storage.  A row whose position is -1
// (padding) is skipped.
#include <float.h>

#include "async_copy.cuh"
#include "common.cuh"

namespace nnis {

template <typename T>
__global__ void __launch_bounds__(256)
qkv_prep_kernel(const float* __restrict__ a, const float* __restrict__ wq, const float* __restrict__ wk,
                const float* __restrict__ freq, const int* __restrict__ token_pos,
                const int* __restrict__ token_seq, const int* __restrict__ page_table, int table_cols,
                T* __restrict__ q_out, T* __restrict__ k_cache, T* __restrict__ v_cache,
                float* __restrict__ gate_out, int H, int G, int dk, int dv, int rot, int gated, int page_size,
                float eps) {
    __shared__ float red[2][8];
    pdl_wait();
    pdl_launch_dependents();
    const int n = blockIdx.x;
    const int pos = token_pos[n];
    if (pos < 0) return;
    const int nq = H * dk, nk = G * dk, nv = G * dv;
    const float* row = a + (size_t)n * (nq + nk + nv + (gated ? H : 0));
    float sq = 0.f, sk = 0.f;
    if (wq) for (int i = threadIdx.x; i < nq; i += 256) sq = fmaf(row[i], row[i], sq);
    if (wk) for (int i = threadIdx.x; i < nk; i += 256) sk = fmaf(row[nq + i], row[nq + i], sk);
    sq = warp_sum(sq);
    sk = warp_sum(sk);
    if ((threadIdx.x & 31) == 0) {
        red[0][threadIdx.x >> 5] = sq;
        red[1][threadIdx.x >> 5] = sk;
    }
    __syncthreads();
    sq = sk = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) {
        sq += red[0][w];
        sk += red[1][w];
    }
    const float inv_q = wq ? 1.0f / sqrtf(sq / (float)nq + eps) : 1.0f;
    const float inv_k = (wk && nk) ? 1.0f / sqrtf(sk / (float)nk + eps) : 1.0f;
    const float p = (float)pos;
    // pairs of q, then pairs of k
    const int pairs_q = nq >> 1, pairs_k = nk >> 1;
    size_t cache_row = 0;
    if (nk) {
        int page = page_table[(size_t)token_seq[n] * table_cols + pos / page_size];
        cache_row = (size_t)page * G * page_size + (pos % page_size);
    }
    for (int i = threadIdx.x; i < pairs_q + pairs_k; i += 256) {
        const bool is_q = i < pairs_q;
        const int e = 2 * (is_q ? i : i - pairs_q);  // element index within q or k
        const float* src = row + (is_q ? 0 : nq) + e;
        const float* wn = is_q ? wq : wk;
        const float inv = is_q ? inv_q : inv_k;
        float x0 = src[0] * inv, x1 = src[1] * inv;
        if (wn) {
            x0 *= wn[e];
            x1 *= wn[e + 1];
        }
        const int head = e / dk, within = e - head * dk;
        if (within < rot) {
            float ang = p * freq[within >> 1];
            float c = cosf(ang), s = sinf(ang);
            float y0 = x0 * c - x1 * s, y1 = x1 * c + x0 * s;
            x0 = y0;
            x1 = y1;
        }
        T* dst = is_q ? q_out + (size_t)n * nq + e
                      : k_cache + (cache_row + (size_t)head * page_size) * dk + within;
        dst[0] = from_float<T>(x0);
        dst[1] = from_float<T>(x1);
    }
    for (int i = threadIdx.x; i < nv; i += 256) {
        const int head = i / dv, within = i - head * dv;
        v_cache[(cache_row + (size_t)head * page_size) * dv + within] = from_float<T>(row[nq + nk + i]);
    }
    if (gated)
        for (int i = threadIdx.x; i < H; i += 256)
            gate_out[(size_t)n * H + i] = 1.0f / (1.0f + expf(-row[nq + nk + nv + i]));
}

// A warp per head of q and of k.  pairing 0: values (2i, 2i + 1) turn together; 1: values (i, i + rot / 2).
template <typename T>
__global__ void __launch_bounds__(256)
qkv_prep_heads_kernel(const float* __restrict__ a, const float* __restrict__ q_scale,
                      const float* __restrict__ freq, const int* __restrict__ token_pos,
                      const int* __restrict__ token_seq, const int* __restrict__ page_table, int table_cols,
                      T* __restrict__ q_out, T* __restrict__ k_cache, T* __restrict__ v_cache,
                      float* __restrict__ gate_out, int H, int G, int dk, int dv, int rot, int pairing,
                      int norm_heads, int gate_cols, int page_size, float eps, int maps, float magnitude) {
    extern __shared__ float turned[];  // [8 warps][dk]
    pdl_wait();
    pdl_launch_dependents();
    const int n = blockIdx.x;
    const int pos = token_pos[n];
    if (pos < 0) return;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nq = H * dk, nk = G * dk, nv = G * dv;
    const float* row = a + (size_t)n * (nq + nk + nv + gate_cols);
    const float p = (float)pos;
    const int half = rot >> 1;
    const int sub = dk / maps;  // the size of one map's vector
    size_t cache_row = 0;
    if (G) {
        int page = page_table[(size_t)token_seq[n] * table_cols + pos / page_size];
        cache_row = (size_t)page * G * page_size + (pos % page_size);
    }
    float* buf = turned + (size_t)warp * dk;
    for (int hh = warp; hh < H + G; hh += 8) {
        const bool is_q = hh < H;
        const int h = is_q ? hh : hh - H;
        const float* src = row + (is_q ? 0 : nq) + (size_t)h * dk;
        // a lane takes a pair: one cosine and one sine serve both of its values, and every map's pair
        // of the same place turns by the same angle
        for (int f = lane; f < half; f += 32) {
            float s, c;
            sincosf(p * freq[f], &s, &c);
            s *= magnitude;
            c *= magnitude;
            for (int base = 0; base < dk; base += sub) {
                const int i0 = base + (pairing ? f : 2 * f), i1 = pairing ? i0 + half : i0 + 1;
                const float x0 = src[i0], x1 = src[i1];
                buf[i0] = x0 * c - x1 * s;
                buf[i1] = x1 * c + x0 * s;
            }
        }
        for (int base = 0; base < dk; base += sub)  // (beyond the rotated values of every map)
            for (int j = rot + lane; j < sub; j += 32) buf[base + j] = src[base + j];
        float inv = 1.0f;
        if (norm_heads) {
            __syncwarp();
            float ss = 0.f;
            for (int i = lane; i < dk; i += 32) ss = fmaf(buf[i], buf[i], ss);
            inv = 1.0f / sqrtf(warp_sum(ss) / (float)dk + eps);
        }
        __syncwarp();
        if (is_q && q_scale) inv *= q_scale[h];
        T* dst = is_q ? q_out + (size_t)n * nq + (size_t)h * dk
                      : k_cache + (cache_row + (size_t)h * page_size) * dk;
        if ((dk & 1) == 0) {  // two values a lane and store (heads start on even places)
            for (int i = 2 * lane; i < dk; i += 64) store2(dst + i, buf[i] * inv, buf[i + 1] * inv);
        } else {
            for (int i = lane; i < dk; i += 32) dst[i] = from_float<T>(buf[i] * inv);
        }
        __syncwarp();  // (the next head's pairs go to the same place)
    }
    for (int i = threadIdx.x; i < nv; i += 256) {
        const int head = i / dv, within = i - head * dv;
        v_cache[(cache_row + (size_t)head * page_size) * dv + within] = from_float<T>(row[nq + nk + i]);
    }
    for (int i = threadIdx.x; i < gate_cols; i += 256)
        gate_out[(size_t)n * gate_cols + i] = 1.0f / (1.0f + expf(-row[nq + nk + nv + i]));
}

// partial record per (token, head, slice): [0] running max, [1] running sum, [2 .. 2 + dv) output
template <typename T, int R>
__global__ void __launch_bounds__(128)
attn_sink_kernel(const T* __restrict__ q, const T* __restrict__ k_cache, const T* __restrict__ v_cache,
                 const int* __restrict__ token_pos, const int* __restrict__ token_seq,
                 const int* __restrict__ page_table, int table_cols, const float* __restrict__ sink,
                 const float* __restrict__ gate, T* __restrict__ out, float* __restrict__ partial,
                 int n_tokens, int nq, int nkv, int dk, int dv, int page_size, int window, int chunk,
                 float scale, float cap, int n_splits, int gate_elems) {
    extern __shared__ float q_smem[];
    pdl_wait();
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int n = blockIdx.x * 4 + warp;
    if (n >= n_tokens) return;
    const int hq = blockIdx.y, split = blockIdx.z;
    const int hk = hq / (nq / nkv);
    const int pos = token_pos[n];
    float* qs = q_smem + warp * dk;

    float m = -FLT_MAX, l = 0.f;
    float acc[R];
#pragma unroll
    for (int r = 0; r < R; ++r) acc[r] = 0.f;
    if (pos < 0) {
        if (n_splits == 1) return;
    } else {
        const T* qrow = q + ((size_t)n * nq + hq) * dk;
        for (int i = lane; i < dk; i += 32) qs[i] = to_float(qrow[i]);
        __syncwarp();
        int lo = window > 0 ? max(0, pos - window + 1) : 0;
        if (chunk > 0) lo = max(lo, (pos / chunk) * chunk);
        const int hi = pos + 1;
        int per = (hi - lo + n_splits - 1) / n_splits;
        per = (per + 31) & ~31;
        const int start = lo + split * per;
        const int end = min(hi, start + per);
        if (sink && split == 0) {  // the sink: a score without a key and without a value
            m = sink[hq];
            l = 1.f;
        }
        const int* table = page_table + (size_t)token_seq[n] * table_cols;
        const float inv_cap = cap > 0.f ? 1.0f / cap : 0.f;
        for (int c = start; c < end; c += 32) {
            const int t = c + lane;
            const bool valid = t < end;
            int row_index = 0;
            float s = -FLT_MAX;
            if (valid) {
                int page = table[t / page_size];
                row_index = (page * nkv + hk) * page_size + (t % page_size);
                const T* krow = k_cache + (size_t)row_index * dk;
                float dot = 0.f;
                const int d4 = (dk & 3) ? 0 : dk;
#pragma unroll 8
                for (int i = 0; i < d4; i += 4) {
                    float4 kv = load4(krow + i);
                    dot = fmaf(qs[i], kv.x, dot);
                    dot = fmaf(qs[i + 1], kv.y, dot);
                    dot = fmaf(qs[i + 2], kv.z, dot);
                    dot = fmaf(qs[i + 3], kv.w, dot);
                }
                for (int i = d4; i < dk; ++i) dot = fmaf(qs[i], to_float(krow[i]), dot);
                s = dot * scale;
                if (cap > 0.f) s = cap * tanhf(s * inv_cap);
            }
            const float m_new = fmaxf(m, warp_max(s));
            const float p = valid ? expf(s - m_new) : 0.f;
            const float alpha = l == 0.f ? 0.f : expf(m - m_new);
            l = l * alpha + warp_sum(p);
            m = m_new;
#pragma unroll
            for (int r = 0; r < R; ++r) acc[r] *= alpha;
            const int count = min(32, end - c);
#pragma unroll 4
            for (int j = 0; j < count; ++j) {
                float pj = __shfl_sync(0xffffffffu, p, j);
                int rj = __shfl_sync(0xffffffffu, row_index, j);
                const T* vrow = v_cache + (size_t)rj * dv;
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    int i = lane + 32 * r;
                    if (i < dv) acc[r] = fmaf(pj, to_float(vrow[i]), acc[r]);
                }
            }
        }
    }
    if (n_splits == 1) {
        float inv = l > 0.f ? 1.0f / l : 0.f;
        const float* ge = (gate && gate_elems > 1) ? gate + ((size_t)n * nq + hq) * dv : nullptr;
        if (gate && !ge) inv *= gate[(size_t)n * nq + hq];
        T* o = out + ((size_t)n * nq + hq) * dv;
#pragma unroll
        for (int r = 0; r < R; ++r) {
            int i = lane + 32 * r;
            if (i < dv) o[i] = from_float<T>(acc[r] * inv * (ge ? ge[i] : 1.0f));
        }
    } else {
        float* rec = partial + (((size_t)n * nq + hq) * n_splits + split) * (size_t)(dv + 2);
        if (lane == 0) {
            rec[0] = m;
            rec[1] = l;
        }
#pragma unroll
        for (int r = 0; r < R; ++r) {
            int i = lane + 32 * r;
            if (i < dv) rec[2 + i] = acc[r];
        }
    }
}

// G query heads of one key/value head in one warp.  q_smem: [4 warps][G][dk] floats.
template <typename T, int R, int G>
__global__ void __launch_bounds__(128)
attn_sink_group_kernel(const T* __restrict__ q, const T* __restrict__ k_cache, const T* __restrict__ v_cache,
                       const int* __restrict__ token_pos, const int* __restrict__ token_seq,
                       const int* __restrict__ page_table, int table_cols, const float* __restrict__ sink,
                       const float* __restrict__ gate, T* __restrict__ out, float* __restrict__ partial,
                       int n_tokens, int nq, int nkv, int dk, int dv, int page_size, int window, int chunk,
                       float scale, float cap, int n_splits, int gate_elems) {
    extern __shared__ __align__(16) float q_smem[];
    pdl_wait();
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int n = blockIdx.x * 4 + warp;
    if (n >= n_tokens) return;
    const int hk = blockIdx.y, split = blockIdx.z;
    const int h0 = hk * G;  // the group's first query head
    const int pos = token_pos[n];
    float* qs = q_smem + (size_t)warp * G * dk;

    float m[G], l[G], acc[G][R];
#pragma unroll
    for (int g = 0; g < G; ++g) {
        m[g] = -FLT_MAX;
        l[g] = 0.f;
#pragma unroll
        for (int r = 0; r < R; ++r) acc[g][r] = 0.f;
    }
    if (pos < 0) {
        if (n_splits == 1) return;
    } else {
        const T* qrow = q + ((size_t)n * nq + h0) * dk;  // the group's heads are neighbours
        for (int i = lane; i < G * dk; i += 32) qs[i] = to_float(qrow[i]);
        __syncwarp();
        int lo = window > 0 ? max(0, pos - window + 1) : 0;
        if (chunk > 0) lo = max(lo, (pos / chunk) * chunk);
        const int hi = pos + 1;
        int per = (hi - lo + n_splits - 1) / n_splits;
        per = (per + 31) & ~31;
        const int start = lo + split * per;
        const int end = min(hi, start + per);
        if (sink && split == 0) {
#pragma unroll
            for (int g = 0; g < G; ++g) {
                m[g] = sink[h0 + g];
                l[g] = 1.f;
            }
        }
        const int* table = page_table + (size_t)token_seq[n] * table_cols;
        const float inv_cap = cap > 0.f ? 1.0f / cap : 0.f;
        const bool by_four = (dk & 3) == 0;
        for (int c = start; c < end; c += 32) {
            const int t = c + lane;
            const bool valid = t < end;
            int row_index = 0;
            float s[G];
#pragma unroll
            for (int g = 0; g < G; ++g) s[g] = 0.f;
            if (valid) {
                int page = table[t / page_size];
                row_index = (page * nkv + hk) * page_size + (t % page_size);
                const T* krow = k_cache + (size_t)row_index * dk;
                if (by_four) {
#pragma unroll 4
                    for (int i = 0; i < dk; i += 4) {
                        const float4 kv = load4(krow + i);
#pragma unroll
                        for (int g = 0; g < G; ++g) {
                            const float4 qv = *reinterpret_cast<const float4*>(qs + g * dk + i);
                            s[g] = fmaf(qv.x, kv.x, s[g]);
                            s[g] = fmaf(qv.y, kv.y, s[g]);
                            s[g] = fmaf(qv.z, kv.z, s[g]);
                            s[g] = fmaf(qv.w, kv.w, s[g]);
                        }
                    }
                } else {
                    for (int i = 0; i < dk; ++i) {
                        const float kv = to_float(krow[i]);
#pragma unroll
                        for (int g = 0; g < G; ++g) s[g] = fmaf(qs[g * dk + i], kv, s[g]);
                    }
                }
            }
            float p[G];
#pragma unroll
            for (int g = 0; g < G; ++g) {
                float sv = s[g] * scale;
                if (cap > 0.f) sv = cap * tanhf(sv * inv_cap);
                sv = valid ? sv : -FLT_MAX;
                const float m_new = fmaxf(m[g], warp_max(sv));
                p[g] = valid ? expf(sv - m_new) : 0.f;
                const float alpha = l[g] == 0.f ? 0.f : expf(m[g] - m_new);
                l[g] = l[g] * alpha + warp_sum(p[g]);
                m[g] = m_new;
#pragma unroll
                for (int r = 0; r < R; ++r) acc[g][r] *= alpha;
            }
            const int count = min(32, end - c);
#pragma unroll 2
            for (int j = 0; j < count; ++j) {
                const int rj = __shfl_sync(0xffffffffu, row_index, j);
                const T* vrow = v_cache + (size_t)rj * dv;
                float vr[R];
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    int i = lane + 32 * r;
                    vr[r] = i < dv ? to_float(vrow[i]) : 0.f;
                }
#pragma unroll
                for (int g = 0; g < G; ++g) {
                    const float pj = __shfl_sync(0xffffffffu, p[g], j);
#pragma unroll
                    for (int r = 0; r < R; ++r) acc[g][r] = fmaf(pj, vr[r], acc[g][r]);
                }
            }
        }
    }
#pragma unroll
    for (int g = 0; g < G; ++g) {
        const int hq = h0 + g;
        if (n_splits == 1) {
            float inv = l[g] > 0.f ? 1.0f / l[g] : 0.f;
            const float* ge = (gate && gate_elems > 1) ? gate + ((size_t)n * nq + hq) * dv : nullptr;
            if (gate && !ge) inv *= gate[(size_t)n * nq + hq];
            T* o = out + ((size_t)n * nq + hq) * dv;
#pragma unroll
            for (int r = 0; r < R; ++r) {
                int i = lane + 32 * r;
                if (i < dv) o[i] = from_float<T>(acc[g][r] * inv * (ge ? ge[i] : 1.0f));
            }
        } else {
            float* rec = partial + (((size_t)n * nq + hq) * n_splits + split) * (size_t)(dv + 2);
            if (lane == 0) {
                rec[0] = m[g];
                rec[1] = l[g];
            }
#pragma unroll
            for (int r = 0; r < R; ++r) {
                int i = lane + 32 * r;
                if (i < dv) rec[2 + i] = acc[g][r];
            }
        }
    }
}

// The slices of a (token, head) added up in ascending order, times the head's gate.
template <typename T>
__global__ void __launch_bounds__(128)
attn_sink_merge_kernel(const float* __restrict__ partial, const float* __restrict__ gate, T* __restrict__ out,
                       int d, int n_splits, int gate_elems) {
    __shared__ float share[64];
    pdl_wait();
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31;
    const size_t row = blockIdx.x;
    const float* rec = partial + row * n_splits * (size_t)(d + 2);
    if (threadIdx.x < 32) {
        float ms[2], ls[2];
        float m = -FLT_MAX;
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            int s = lane + 32 * k;
            ms[k] = s < n_splits ? rec[(size_t)s * (d + 2)] : 0.f;
            ls[k] = s < n_splits ? rec[(size_t)s * (d + 2) + 1] : 0.f;
            if (ls[k] > 0.f) m = fmaxf(m, ms[k]);
        }
        m = warp_max(m);
        float l = 0.f;
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            ms[k] = ls[k] > 0.f ? expf(ms[k] - m) : 0.f;
            l += ls[k] * ms[k];
        }
        l = warp_sum(l);
        float inv = l > 0.f ? 1.0f / l : 0.f;
        if (gate && gate_elems <= 1) inv *= gate[row];
        share[lane] = ms[0] * inv;
        share[lane + 32] = ms[1] * inv;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < d; i += 128) {
        float o = 0.f;
        for (int s = 0; s < n_splits; ++s) {
            float w = share[s];
            if (w > 0.f) o = fmaf(w, rec[(size_t)s * (d + 2) + 2 + i], o);
        }
        if (gate && gate_elems > 1) o *= gate[row * d + i];
        out[row * d + i] = from_float<T>(o);
    }
}

template <typename T>
static int launch_attn_sink(const void* q, const void* k_cache, const void* v_cache, const int* token_pos,
                            const int* token_seq, const int* page_table, int table_cols, const float* sink,
                            const float* gate, void* out, float* partial, int n_tokens, int nq, int nkv, int dk,
                            int dv, int page_size, int window, int chunk, float scale, float cap, int n_splits,
                            int gate_elems, cudaStream_t stream) {
    cudaError_t e;
    const int group = nq / nkv;
    const size_t group_smem = 4 * (size_t)group * dk * sizeof(float);
    if ((group == 2 || group == 3 || group == 4 || group == 6 || group == 8) && dv <= 128 &&
        group_smem <= 48 * 1024 && nkv <= 65535) {
        dim3 ggrid((n_tokens + 3) / 4, nkv, n_splits);
#define NNIS_GROUP_CASE(R, G) \
    e = launch_dependent(attn_sink_group_kernel<T, R, G>, ggrid, 128, group_smem, stream, (const T*)q, \
                         (const T*)k_cache, (const T*)v_cache, token_pos, token_seq, page_table, table_cols, sink, \
                         gate, (T*)out, partial, n_tokens, nq, nkv, dk, dv, page_size, window, chunk, scale, cap, \
                         n_splits, gate_elems)
#define NNIS_GROUP_R(G) \
    if (dv <= 32) NNIS_GROUP_CASE(1, G); \
    else if (dv <= 64) NNIS_GROUP_CASE(2, G); \
    else NNIS_GROUP_CASE(4, G)
        if (group == 2) { NNIS_GROUP_R(2); }
        else if (group == 3) { NNIS_GROUP_R(3); }
        else if (group == 4) { NNIS_GROUP_R(4); }
        else if (group == 6) { NNIS_GROUP_R(6); }
        else { NNIS_GROUP_R(8); }
#undef NNIS_GROUP_R
#undef NNIS_GROUP_CASE
        if (e != cudaSuccess) return (int)e;
        if (n_splits > 1) {
            size_t rows = (size_t)n_tokens * nq;
            e = launch_dependent(attn_sink_merge_kernel<T>, (unsigned)rows, 128, 0, stream, (const float*)partial,
                                 gate, (T*)out, dv, n_splits, gate_elems);
        }
        return e == cudaSuccess ? NNIS_OK : (int)e;
    }
    dim3 grid((n_tokens + 3) / 4, nq, n_splits);
    size_t smem = 4 * (size_t)dk * sizeof(float);
#define NNIS_SINK_CASE(R) \
    e = launch_dependent(attn_sink_kernel<T, R>, grid, 128, smem, stream, (const T*)q, (const T*)k_cache, \
                         (const T*)v_cache, token_pos, token_seq, page_table, table_cols, sink, gate, (T*)out, \
                         partial, n_tokens, nq, nkv, dk, dv, page_size, window, chunk, scale, cap, n_splits, \
                         gate_elems)
    if (dv <= 32) NNIS_SINK_CASE(1);
    else if (dv <= 64) NNIS_SINK_CASE(2);
    else if (dv <= 128) NNIS_SINK_CASE(4);
    else NNIS_SINK_CASE(8);
#undef NNIS_SINK_CASE
    if (e != cudaSuccess) return (int)e;
    if (n_splits > 1) {
        size_t rows = (size_t)n_tokens * nq;
        e = launch_dependent(attn_sink_merge_kernel<T>, (unsigned)rows, 128, 0, stream, (const float*)partial, gate,
                             (T*)out, dv, n_splits, gate_elems);
    }
    return e == cudaSuccess ? NNIS_OK : (int)e;
}

}  // namespace nnis

using namespace nnis;

// a: float32 [n, H dk + G dk + G dv + (gated ? H : 0)] with G = 0 for rows without keys and values;
// wq, wk: float32 norm weights or null; freq: float32 [rot / 2]
NNIS_API int nnis_qkv_prep(const float* a, const float* wq, const float* wk, const float* freq,
                           const int* token_pos, const int* token_seq, const int* page_table, int table_cols,
                           void* q_out, void* k_cache, void* v_cache, float* gate_out, int n_tokens, int H, int G,
                           int dk, int dv, int rot, int gated, int page_size, float eps, int dtype,
                           cudaStream_t stream) {
    if (n_tokens <= 0 || H <= 0 || G < 0 || dk <= 0 || dv <= 0 || rot < 0 || !a || !q_out || !token_pos)
        return NNIS_ERR_ARGUMENT;
    if ((dk & 1) || (rot & 1) || rot > dk) return NNIS_ERR_UNSUPPORTED;
    if (rot > 0 && !freq) return NNIS_ERR_ARGUMENT;
    if (G > 0 && (!k_cache || !v_cache || !page_table || !token_seq || page_size <= 0)) return NNIS_ERR_ARGUMENT;
    if (gated && !gate_out) return NNIS_ERR_ARGUMENT;
    cudaError_t e;
    if (dtype == NNIS_DTYPE_F32)
        e = launch_dependent(qkv_prep_kernel<float>, (unsigned)n_tokens, 256, 0, stream, a, wq, wk, freq, token_pos,
                             token_seq, page_table, table_cols, (float*)q_out, (float*)k_cache, (float*)v_cache,
                             gate_out, H, G, dk, dv, rot, gated, page_size, eps);
    else if (dtype == NNIS_DTYPE_BF16)
        e = launch_dependent(qkv_prep_kernel<bf16>, (unsigned)n_tokens, 256, 0, stream, a, wq, wk, freq, token_pos,
                             token_seq, page_table, table_cols, (bf16*)q_out, (bf16*)k_cache, (bf16*)v_cache,
                             gate_out, H, G, dk, dv, rot, gated, page_size, eps);
    else
        return NNIS_ERR_UNSUPPORTED;
    return e == cudaSuccess ? NNIS_OK : (int)e;
}

// a: float32 [n, H dk + G dk + G dv + gate_cols]; q_scale: float32 [H] or null; pairing 0: neighbours,
// 1: halves; norm_heads: every q and k head divided by its own root mean square after the rotation;
// maps: vectors of dk / maps values side by side in a head, each turned by itself; magnitude: a
// multiplier of every cosine and sine
NNIS_API int nnis_qkv_prep_heads(const float* a, const float* q_scale, const float* freq, const int* token_pos,
                                 const int* token_seq, const int* page_table, int table_cols, void* q_out,
                                 void* k_cache, void* v_cache, float* gate_out, int n_tokens, int H, int G, int dk,
                                 int dv, int rot, int pairing, int norm_heads, int gate_cols, int page_size,
                                 float eps, int maps, float magnitude, int dtype, cudaStream_t stream) {
    if (n_tokens <= 0 || H <= 0 || G < 0 || dk <= 0 || dv <= 0 || rot < 0 || gate_cols < 0 || !a || !q_out ||
        !token_pos)
        return NNIS_ERR_ARGUMENT;
    if (maps <= 0 || dk % maps) return NNIS_ERR_ARGUMENT;
    if ((rot & 1) || rot > dk / maps || dk > 1024 || ((dk / maps) & 1 && maps > 1 && !pairing))
        return NNIS_ERR_UNSUPPORTED;
    if (rot > 0 && !freq) return NNIS_ERR_ARGUMENT;
    if (G > 0 && (!k_cache || !v_cache || !page_table || !token_seq || page_size <= 0)) return NNIS_ERR_ARGUMENT;
    if (gate_cols && !gate_out) return NNIS_ERR_ARGUMENT;
    const size_t smem = 8 * (size_t)dk * sizeof(float);
    cudaError_t e;
    if (dtype == NNIS_DTYPE_F32)
        e = launch_dependent(qkv_prep_heads_kernel<float>, (unsigned)n_tokens, 256, smem, stream, a, q_scale, freq,
                             token_pos, token_seq, page_table, table_cols, (float*)q_out, (float*)k_cache,
                             (float*)v_cache, gate_out, H, G, dk, dv, rot, pairing, norm_heads, gate_cols, page_size,
                             eps, maps, magnitude);
    else if (dtype == NNIS_DTYPE_BF16)
        e = launch_dependent(qkv_prep_heads_kernel<bf16>, (unsigned)n_tokens, 256, smem, stream, a, q_scale, freq,
                             token_pos, token_seq, page_table, table_cols, (bf16*)q_out, (bf16*)k_cache,
                             (bf16*)v_cache, gate_out, H, G, dk, dv, rot, pairing, norm_heads, gate_cols, page_size,
                             eps, maps, magnitude);
    else
        return NNIS_ERR_UNSUPPORTED;
    return e == cudaSuccess ? NNIS_OK : (int)e;
}

// q: [n, nq * dk]; caches [pages, nkv, page, dk] and [pages, nkv, page, dv]; sink: float32 [nq] or
// null; gate: float32 [n, nq] (gate_elems 0 or 1) or [n, nq * dv] (gate_elems = dv) or null; partial:
// n * nq * n_splits * (dv + 2) floats when n_splits > 1
NNIS_API int nnis_attention_sink(const void* q, const void* k_cache, const void* v_cache, const int* token_pos,
                                 const int* token_seq, const int* page_table, int table_cols, const float* sink,
                                 const float* gate, void* out, float* partial, int n_tokens, int nq, int nkv,
                                 int dk, int dv, int page_size, int window, int chunk, float scale, float cap,
                                 int n_splits, int gate_elems, int dtype, cudaStream_t stream) {
    if (n_tokens <= 0 || nq <= 0 || nkv <= 0 || nq % nkv || page_size <= 0 || table_cols <= 0 || n_splits <= 0 ||
        window < 0 || chunk < 0 || cap < 0.f)
        return NNIS_ERR_ARGUMENT;
    if (dk <= 0 || dv <= 0 || dk > 1024 || dv > 256) return NNIS_ERR_UNSUPPORTED;
    if (nq > 65535 || n_splits > 64) return NNIS_ERR_UNSUPPORTED;
    if (n_splits > 1 && !partial) return NNIS_ERR_ARGUMENT;
    if (gate_elems > 1 && gate_elems != dv) return NNIS_ERR_ARGUMENT;
    if (dtype == NNIS_DTYPE_F32)
        return launch_attn_sink<float>(q, k_cache, v_cache, token_pos, token_seq, page_table, table_cols, sink, gate,
                                       out, partial, n_tokens, nq, nkv, dk, dv, page_size, window, chunk, scale,
                                       cap, n_splits, gate_elems, stream);
    if (dtype == NNIS_DTYPE_BF16)
        return launch_attn_sink<bf16>(q, k_cache, v_cache, token_pos, token_seq, page_table, table_cols, sink, gate,
                                      out, partial, n_tokens, nq, nkv, dk, dv, page_size, window, chunk, scale,
                                      cap, n_splits, gate_elems, stream);
    return NNIS_ERR_UNSUPPORTED;
}
