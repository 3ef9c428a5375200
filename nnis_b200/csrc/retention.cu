// Retention: linear attention with a fixed decay per head, no softmax and no
// denominator.  Per head, with q and k rotated by position and k scaled by
// dim^-1/2:   S_t = g S_{t-1} + k_t v_t^T,   o_t = S_t^T q_t.
// The state S [dim, vdim] lives in float32 in a per-sequence state area and is
// carried from step to step; everything between the projections and the output
// (angles, rotation, decay, state, the head's unit norm, the gate) is float32.
//
//   retention_scan   a CTA per (sequence, head, 32 columns of vdim) walks the step's
//                    tokens of that sequence in order; warp w holds rows w, w+8, ...
//                    of the state tile in registers.  Steps of single tokens.
//   retention_chunk  prompts and later chunks of them (the state says where a sequence
//                    stands): 32 tokens at a time, see below.
//   retention_prefix, retention_carry   long prompts cut into runs that are worked side by
//                    side: the states between the runs, and what they give each token.
//   retention_gate   o / rms(o) per head, times silu(g) (or sigmoid(g)), rounded once;
//   retention_gate_joined   the same with one norm over a token's joined heads and a weight per value.
//
// `act` passes q, k and v through silu as they are read; `k_scale` multiplies k (dim^-1/2 in
// retention proper, 1 for a recurrence without a scale).
//
// Packed input rows: [q (H dim) | k (H dim) | v (H vdim) | g (H vdim)].
#include "async_copy.cuh"
#include "common.cuh"

namespace nnis {

// a projection's value as it enters the recurrence: as it is, or through silu (`act`)
template <typename T> __device__ __forceinline__ float pre(T x, int act) {
    const float f = to_float(x);
    return act ? f / (1.0f + expf(-f)) : f;
}

template <typename T, int R>
__global__ void __launch_bounds__(256)
retention_scan_kernel(const T* __restrict__ qkvg, const float* __restrict__ freq,
                      const float* __restrict__ decay, float* __restrict__ state,
                      const int* __restrict__ token_pos, const int* __restrict__ token_seq,
                      const int* __restrict__ seq_slots, const int* __restrict__ seq_first_row,
                      const int* __restrict__ seq_start, const int* __restrict__ seq_count,
                      float* __restrict__ o_raw, int heads, int dim, int vdim, int rot_dims, int act, float k_scale) {
    extern __shared__ float smem[];
    pdl_wait();
    pdl_launch_dependents();
    float* qs = smem;             // [dim]
    float* ks = smem + dim;       // [dim]
    float* red = smem + 2 * dim;  // [8][32]
    int unit = blockIdx.x, h = blockIdx.y, col = blockIdx.z * 32 + (threadIdx.x & 31);
    int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int first, start, count, slot;
    if (seq_first_row) {
        first = seq_first_row[unit];
        start = seq_start[unit];
        count = seq_count[unit];
        slot = seq_slots[unit];
    } else {  // one token per row; a row without a sequence has position -1
        first = unit;
        start = token_pos[unit];
        count = start < 0 ? 0 : 1;
        slot = seq_slots[token_seq[unit]];
    }
    if (count <= 0) return;
    const bool live = col < vdim;
    const float g = decay[h];
    float* S = state + (((size_t)slot * heads + h) * dim) * vdim;
    float s[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
        int i = warp + 8 * r;
        s[r] = (live && i < dim) ? S[(size_t)i * vdim + col] : 0.f;
    }
    const size_t row_len = (size_t)2 * heads * dim + (size_t)2 * heads * vdim;
    const int half = rot_dims >> 1;
    for (int t = 0; t < count; ++t) {
        const T* row = qkvg + (size_t)(first + t) * row_len;
        const T* qh = row + (size_t)h * dim;
        const T* kh = row + (size_t)heads * dim + (size_t)h * dim;
        float pos = (float)(start + t);
        for (int j = threadIdx.x; j < dim - half; j += 256) {
            if (j < half) {
                float ang = pos * freq[j];
                float c = cosf(ang), sn = sinf(ang);
                float u = pre(qh[j], act), v = pre(qh[j + half], act);
                qs[j] = u * c - v * sn;
                qs[j + half] = v * c + u * sn;
                u = pre(kh[j], act);
                v = pre(kh[j + half], act);
                ks[j] = (u * c - v * sn) * k_scale;
                ks[j + half] = (v * c + u * sn) * k_scale;
            } else {
                qs[j + half] = pre(qh[j + half], act);
                ks[j + half] = pre(kh[j + half], act) * k_scale;
            }
        }
        __syncthreads();
        float v = live ? pre(row[(size_t)2 * heads * dim + (size_t)h * vdim + col], act) : 0.f;
        float o = 0.f;
#pragma unroll
        for (int r = 0; r < R; ++r) {
            int i = warp + 8 * r;
            if (i < dim) {
                s[r] = fmaf(g, s[r], ks[i] * v);
                o = fmaf(s[r], qs[i], o);
            }
        }
        red[warp * 32 + lane] = o;
        __syncthreads();
        if (warp == 0 && live) {
            float sum = 0.f;
#pragma unroll
            for (int w = 0; w < 8; ++w) sum += red[w * 32 + lane];
            o_raw[((size_t)(first + t) * heads + h) * vdim + col] = sum;
        }
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
        int i = warp + 8 * r;
        if (live && i < dim) S[(size_t)i * vdim + col] = s[r];
    }
}

// Prompts: the same recurrence a chunk of 32 tokens at a time.  Within a chunk, with
// A[i][j] = (q_i . k_j) g^(i-j) for j <= i:
//     o_i = sum_j A[i][j] v_j + g^(i+1) S^T q_i        S <- g^C S + sum_j g^(C-1-j) k_j v_j^T
// (C tokens in the chunk, S the state before it), all in float32 on the CUDA cores.  A CTA
// owns (sequence, head, 32 columns of vdim) and walks the chunks in order with its tile of
// S in shared memory; q and k of the chunk are rotated once into shared memory.
constexpr int kRetChunk = 32;

// DR4: dim / 32 (the kernel takes dim = 32, 64, 128, 256; a warp owns dim / 8 rows of the
// state in the update).  The three products are tiled in registers: 2 x 2 entries of A per
// thread, four rows of the output per thread, dim / 8 rows of the state per thread, with
// q and k read as float4 along dim.
template <typename T, int DR4>
__global__ void __launch_bounds__(256)
retention_chunk_kernel(const T* __restrict__ qkvg, const float* __restrict__ freq,
                       const float* __restrict__ decay, float* __restrict__ state,
                       const int* __restrict__ seq_slots, const int* __restrict__ seq_first_row,
                       const int* __restrict__ seq_start, const int* __restrict__ seq_count,
                       const int* __restrict__ segments, int seg_len, float* __restrict__ seg_state,
                       float* __restrict__ o_raw, int heads, int vdim, int rot_dims, int act, float k_scale) {
    constexpr int C = kRetChunk, dim = 32 * DR4, ld = dim + 4, DR = 4 * DR4;
    extern __shared__ __align__(16) float smem[];
    float* qs = smem;                  // [C][dim + 4]
    float* ks = qs + C * ld;           // [C][dim + 4]
    float* Ss = ks + C * ld;           // [dim][32]
    float* As = Ss + dim * 32;         // [C][C + 1]
    float* vs = As + C * (C + 1);      // [C][32]
    float* pw = vs + C * 32;           // [C + 1]: g^n
    const int h = blockIdx.y;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, tid = threadIdx.x;
    const int col = blockIdx.z * 32 + lane;
    // a unit is a sequence, from and into its state; or, with `segments`, a run of seg_len
    // tokens of a sequence from a zero state into a state of its own (retention_carry adds
    // what the tokens before the run contribute)
    const int unit = segments ? segments[2 * blockIdx.x] : (int)blockIdx.x;
    const int begin = segments ? segments[2 * blockIdx.x + 1] : 0;
    const int first = seq_first_row[unit] + begin, start = seq_start[unit] + begin;
    const int count = segments ? min(seg_len, seq_count[unit] - begin) : seq_count[unit];
    if (count <= 0) return;
    const bool live = col < vdim;
    const float g = decay[h];
    float* S = segments ? seg_state + (((size_t)blockIdx.x * heads + h) * dim) * vdim
                        : state + (((size_t)seq_slots[unit] * heads + h) * dim) * vdim;
    for (int d = warp; d < dim; d += 8) Ss[d * 32 + lane] = live && !segments ? S[(size_t)d * vdim + col] : 0.f;
    for (int it = tid; it < 2 * C * ld; it += 256) qs[it] = 0.f;  // (rows beyond a short chunk)
    if (tid == 0) {
        float p = 1.f;
        for (int n = 0; n <= C; ++n) {
            pw[n] = p;
            p *= g;
        }
    }
    const size_t row_len = (size_t)2 * heads * dim + (size_t)2 * heads * vdim;
    const int half = rot_dims >> 1, per_tok = dim - half;
    for (int t0 = 0; t0 < count; t0 += C) {
        const int cnt = min(C, count - t0);
        __syncthreads();  // the chunk before is done with qs, ks, vs, As; Ss is up to date
        for (int it = tid; it < cnt * per_tok; it += 256) {
            int i = it / per_tok, j = it - i * per_tok;
            const T* row = qkvg + (size_t)(first + t0 + i) * row_len;
            const T* qh = row + (size_t)h * dim;
            const T* kh = row + (size_t)heads * dim + (size_t)h * dim;
            if (j < half) {
                float ang = (float)(start + t0 + i) * freq[j];
                float c = cosf(ang), sn = sinf(ang);
                float u = pre(qh[j], act), v = pre(qh[j + half], act);
                qs[i * ld + j] = u * c - v * sn;
                qs[i * ld + j + half] = v * c + u * sn;
                u = pre(kh[j], act);
                v = pre(kh[j + half], act);
                ks[i * ld + j] = (u * c - v * sn) * k_scale;
                ks[i * ld + j + half] = (v * c + u * sn) * k_scale;
            } else {
                qs[i * ld + j + half] = pre(qh[j + half], act);
                ks[i * ld + j + half] = pre(kh[j + half], act) * k_scale;
            }
        }
        for (int it = tid; it < C * 32; it += 256) {
            int i = it >> 5;
            float v = 0.f;
            if (i < cnt && live)
                v = pre(qkvg[(size_t)(first + t0 + i) * row_len + (size_t)2 * heads * dim +
                             (size_t)h * vdim + col], act);
            vs[it] = v;
        }
        __syncthreads();
        {   // A[i][j] = (q_i . k_j) g^(i - j) for j <= i: a 2 x 2 tile per thread
            const int i0 = (tid >> 4) * 2, j0 = (tid & 15) * 2;
            float a00 = 0.f, a01 = 0.f, a10 = 0.f, a11 = 0.f;
            if (j0 <= i0 + 1) {
                const float4* q0 = reinterpret_cast<const float4*>(qs + i0 * ld);
                const float4* q1 = reinterpret_cast<const float4*>(qs + (i0 + 1) * ld);
                const float4* k0 = reinterpret_cast<const float4*>(ks + j0 * ld);
                const float4* k1 = reinterpret_cast<const float4*>(ks + (j0 + 1) * ld);
#pragma unroll 4
                for (int d = 0; d < dim / 4; ++d) {
                    float4 x0 = q0[d], x1 = q1[d], y0 = k0[d], y1 = k1[d];
                    a00 = fmaf(x0.x, y0.x, fmaf(x0.y, y0.y, fmaf(x0.z, y0.z, fmaf(x0.w, y0.w, a00))));
                    a01 = fmaf(x0.x, y1.x, fmaf(x0.y, y1.y, fmaf(x0.z, y1.z, fmaf(x0.w, y1.w, a01))));
                    a10 = fmaf(x1.x, y0.x, fmaf(x1.y, y0.y, fmaf(x1.z, y0.z, fmaf(x1.w, y0.w, a10))));
                    a11 = fmaf(x1.x, y1.x, fmaf(x1.y, y1.y, fmaf(x1.z, y1.z, fmaf(x1.w, y1.w, a11))));
                }
            }
            As[i0 * (C + 1) + j0] = j0 <= i0 ? a00 * pw[i0 - j0] : 0.f;
            As[i0 * (C + 1) + j0 + 1] = j0 + 1 <= i0 ? a01 * pw[i0 - j0 - 1] : 0.f;
            As[(i0 + 1) * (C + 1) + j0] = j0 <= i0 + 1 ? a10 * pw[i0 + 1 - j0] : 0.f;
            As[(i0 + 1) * (C + 1) + j0 + 1] = j0 <= i0 ? a11 * pw[i0 - j0] : 0.f;
        }
        __syncthreads();
        {   // outputs: rows 4 warp .. 4 warp + 3, column = lane
            const int i0 = warp * 4;
            float inter[4] = {0.f, 0.f, 0.f, 0.f}, intra[4] = {0.f, 0.f, 0.f, 0.f};
            if (i0 < cnt) {
#pragma unroll 2
                for (int d = 0; d < dim; d += 4) {
                    float s0 = Ss[d * 32 + lane], s1 = Ss[(d + 1) * 32 + lane];
                    float s2 = Ss[(d + 2) * 32 + lane], s3 = Ss[(d + 3) * 32 + lane];
#pragma unroll
                    for (int r = 0; r < 4; ++r) {
                        float4 x = *reinterpret_cast<const float4*>(qs + (i0 + r) * ld + d);
                        inter[r] = fmaf(x.x, s0, fmaf(x.y, s1, fmaf(x.z, s2, fmaf(x.w, s3, inter[r]))));
                    }
                }
                for (int j = 0; j <= i0 + 3; ++j) {  // (A is zero above its diagonal)
                    float v = vs[j * 32 + lane];
#pragma unroll
                    for (int r = 0; r < 4; ++r) intra[r] = fmaf(As[(i0 + r) * (C + 1) + j], v, intra[r]);
                }
#pragma unroll
                for (int r = 0; r < 4; ++r)
                    if (live && i0 + r < cnt)
                        o_raw[((size_t)(first + t0 + i0 + r) * heads + h) * vdim + col] =
                            fmaf(pw[i0 + r + 1], inter[r], intra[r]);
            }
        }
        __syncthreads();
        {   // the state after the chunk: rows warp * DR .. + DR - 1, column = lane
            const int d0 = warp * DR;
            float acc[DR];
#pragma unroll
            for (int r = 0; r < DR; ++r) acc[r] = 0.f;
            for (int j = 0; j < cnt; ++j) {
                float v = pw[cnt - 1 - j] * vs[j * 32 + lane];
#pragma unroll
                for (int r4 = 0; r4 < DR4; ++r4) {
                    float4 k = *reinterpret_cast<const float4*>(ks + j * ld + d0 + 4 * r4);
                    acc[4 * r4] = fmaf(k.x, v, acc[4 * r4]);
                    acc[4 * r4 + 1] = fmaf(k.y, v, acc[4 * r4 + 1]);
                    acc[4 * r4 + 2] = fmaf(k.z, v, acc[4 * r4 + 2]);
                    acc[4 * r4 + 3] = fmaf(k.w, v, acc[4 * r4 + 3]);
                }
            }
#pragma unroll
            for (int r = 0; r < DR; ++r) Ss[(d0 + r) * 32 + lane] = fmaf(pw[cnt], Ss[(d0 + r) * 32 + lane], acc[r]);
        }
    }
    __syncthreads();
    for (int d = warp; d < dim; d += 8)
        if (live) S[(size_t)d * vdim + col] = Ss[d * 32 + lane];
}

// Long prompts run as runs of seg_len tokens side by side (retention_chunk with `segments`),
// each from a zero state.  This kernel then walks a sequence's runs in order, per element of
// the state: the state before a run replaces the run's own in `seg_state`, and the state
// after the last run goes to the sequence's slot.  S_before(r + 1) = g^len(r) S_before(r) + U(r).
__global__ void __launch_bounds__(256)
retention_prefix_kernel(float* __restrict__ seg_state, float* __restrict__ state,
                        const float* __restrict__ decay, const int* __restrict__ seq_slots,
                        const int* __restrict__ seq_count, const int* __restrict__ seq_first_segment,
                        int seg_len, int heads, int per_head) {
    const int b = blockIdx.x, h = blockIdx.y;
    const int e = blockIdx.z * 256 + threadIdx.x;
    if (e >= per_head) return;
    const int s0 = seq_first_segment[b], s1 = seq_first_segment[b + 1], count = seq_count[b];
    const float g = decay[h];
    float* cell = state + ((size_t)seq_slots[b] * heads + h) * per_head + e;
    float run = *cell;
    // g^32 and g^seg_len as the chunk kernel's chain of products makes them
    float g32 = 1.f;
    for (int n = 0; n < 32; ++n) g32 *= g;
    float g_run = 1.f;
    for (int n = 0; n < seg_len / 32; ++n) g_run *= g32;
    for (int s = s0; s < s1; ++s) {
        int len = min(seg_len, count - (s - s0) * seg_len);
        float p = g_run;
        if (len < seg_len) {  // the last, shorter run: whole chunks, then the rest
            p = 1.f;
            for (int n = 0; n < len / 32; ++n) p *= g32;
            float rest = 1.f;
            for (int n = 0; n < len % 32; ++n) rest *= g;
            p *= rest;
        }
        float* u = seg_state + ((size_t)s * heads + h) * per_head + e;
        float after = fmaf(p, run, *u);
        *u = run;
        run = after;
    }
    *cell = run;
}

// ... and this one adds to every token of a run what the state before the run gives it:
// o_i += g^(i + 1) S_before^T q_i, i counted within the run.
template <typename T, int DR4>
__global__ void __launch_bounds__(256)
retention_carry_kernel(const T* __restrict__ qkvg, const float* __restrict__ freq,
                       const float* __restrict__ decay, const float* __restrict__ seg_state,
                       const int* __restrict__ seq_first_row, const int* __restrict__ seq_start,
                       const int* __restrict__ seq_count, const int* __restrict__ segments, int seg_len,
                       float* __restrict__ o_raw, int heads, int vdim, int rot_dims, int act, float k_scale) {
    constexpr int C = kRetChunk, dim = 32 * DR4, ld = dim + 4;
    extern __shared__ __align__(16) float smem[];
    float* qs = smem;             // [C][dim + 4]
    float* Ss = qs + C * ld;      // [dim][32]
    float* pw = Ss + dim * 32;    // [seg_len + 1]
    const int h = blockIdx.y, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, tid = threadIdx.x;
    const int col = blockIdx.z * 32 + lane;
    const int unit = segments[2 * blockIdx.x], begin = segments[2 * blockIdx.x + 1];
    const int first = seq_first_row[unit] + begin, start = seq_start[unit] + begin;
    const int count = min(seg_len, seq_count[unit] - begin);
    if (count <= 0 || (begin == 0 && seq_start[unit] == 0)) return;  // (nothing before a sequence's start)
    const bool live = col < vdim;
    const float* S = seg_state + (((size_t)blockIdx.x * heads + h) * dim) * vdim;
    for (int d = warp; d < dim; d += 8) Ss[d * 32 + lane] = live ? S[(size_t)d * vdim + col] : 0.f;
    for (int it = tid; it < C * ld; it += 256) qs[it] = 0.f;
    if (tid == 0) {
        float p = 1.f, g = decay[h];
        for (int n = 0; n <= seg_len; ++n) {
            pw[n] = p;
            p *= g;
        }
    }
    const size_t row_len = (size_t)2 * heads * dim + (size_t)2 * heads * vdim;
    const int half = rot_dims >> 1, per_tok = dim - half;
    for (int t0 = 0; t0 < count; t0 += C) {
        const int cnt = min(C, count - t0);
        __syncthreads();
        for (int it = tid; it < cnt * per_tok; it += 256) {
            int i = it / per_tok, j = it - i * per_tok;
            const T* qh = qkvg + (size_t)(first + t0 + i) * row_len + (size_t)h * dim;
            if (j < half) {
                float ang = (float)(start + t0 + i) * freq[j];
                float c = cosf(ang), sn = sinf(ang);
                float u = pre(qh[j], act), v = pre(qh[j + half], act);
                qs[i * ld + j] = u * c - v * sn;
                qs[i * ld + j + half] = v * c + u * sn;
            } else {
                qs[i * ld + j + half] = pre(qh[j + half], act);
            }
        }
        __syncthreads();
        const int i0 = warp * 4;
        if (i0 < cnt) {
            float inter[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 2
            for (int d = 0; d < dim; d += 4) {
                float s0 = Ss[d * 32 + lane], s1 = Ss[(d + 1) * 32 + lane];
                float s2 = Ss[(d + 2) * 32 + lane], s3 = Ss[(d + 3) * 32 + lane];
#pragma unroll
                for (int r = 0; r < 4; ++r) {
                    float4 x = *reinterpret_cast<const float4*>(qs + (i0 + r) * ld + d);
                    inter[r] = fmaf(x.x, s0, fmaf(x.y, s1, fmaf(x.z, s2, fmaf(x.w, s3, inter[r]))));
                }
            }
#pragma unroll
            for (int r = 0; r < 4; ++r)
                if (live && i0 + r < cnt) {
                    float* o = o_raw + ((size_t)(first + t0 + i0 + r) * heads + h) * vdim + col;
                    *o = fmaf(pw[t0 + i0 + r + 1], inter[r], *o);
                }
        }
    }
}

// out[n, h, :] = o[n, h, :] / sqrt(mean(o[n, h, :]^2) + eps) * silu(g[n, h, :]); a warp
// per (token, head); a row at position -1 is left alone
template <typename T>
__global__ void __launch_bounds__(256)
retention_gate_kernel(const float* __restrict__ o_raw, const T* __restrict__ qkvg,
                      const int* __restrict__ token_pos, T* __restrict__ out, long long n_units,
                      int heads, int dim, int vdim, float eps, int gate_kind) {
    pdl_wait();
    pdl_launch_dependents();
    long long unit = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (unit >= n_units) return;
    int lane = threadIdx.x & 31;
    long long n = unit / heads;
    int h = (int)(unit - n * heads);
    T* dst = out + (size_t)unit * vdim;
    if (token_pos[n] < 0) {
        for (int i = lane; i < vdim; i += 32) dst[i] = from_float<T>(0.f);
        return;
    }
    const float* o = o_raw + (size_t)unit * vdim;
    const T* gate = qkvg + (size_t)n * ((size_t)2 * heads * dim + (size_t)2 * heads * vdim) +
                    (size_t)2 * heads * dim + (size_t)heads * vdim + (size_t)h * vdim;
    float ss = 0.f;
    for (int i = lane; i < vdim; i += 32) ss = fmaf(o[i], o[i], ss);
    ss = warp_sum(ss);
    float s = 1.0f / sqrtf(ss / (float)vdim + eps);
    for (int i = lane; i < vdim; i += 32) {
        float z = to_float(gate[i]);
        float sg = 1.0f / (1.0f + expf(-z));
        dst[i] = from_float<T>((o[i] * s) * (gate_kind ? sg : z * sg));
    }
}

// The same with ONE norm over the joined heads of a token and a weight per value:
// out[n, :] = o[n, :] / sqrt(mean(o[n, :]^2) + eps) * w * gate(g[n, :]); a CTA per token
template <typename T>
__global__ void __launch_bounds__(256)
retention_gate_joined_kernel(const float* __restrict__ o_raw, const T* __restrict__ qkvg,
                             const float* __restrict__ w, const int* __restrict__ token_pos, T* __restrict__ out,
                             int heads, int dim, int vdim, float eps, int gate_kind) {
    __shared__ float red[8];
    pdl_wait();
    pdl_launch_dependents();
    const size_t n = blockIdx.x;
    const int cols = heads * vdim;
    T* dst = out + n * cols;
    if (token_pos[n] < 0) {
        for (int i = threadIdx.x; i < cols; i += 256) dst[i] = from_float<T>(0.f);
        return;
    }
    const float* o = o_raw + n * cols;
    const T* gate = qkvg + n * ((size_t)2 * heads * dim + (size_t)2 * cols) + (size_t)2 * heads * dim + cols;
    float ss = 0.f;
    for (int i = threadIdx.x; i < cols; i += 256) ss = fmaf(o[i], o[i], ss);
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float total = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) total += red[k];
    const float s = 1.0f / sqrtf(total / (float)cols + eps);
    for (int i = threadIdx.x; i < cols; i += 256) {
        float z = to_float(gate[i]);
        float sg = 1.0f / (1.0f + expf(-z));
        dst[i] = from_float<T>((o[i] * s) * w[i] * (gate_kind ? sg : z * sg));
    }
}

template <typename T>
static int launch_retention(const void* qkvg, const float* freq, const float* decay, float* state,
                            const int* token_pos, const int* token_seq, const int* seq_slots,
                            const int* seq_first_row, const int* seq_start, const int* seq_count,
                            const int* segments, int n_segments, const int* seq_first_segment, int seg_len,
                            float* seg_state, float* o_raw, void* out, int n_tokens, int n_units, int heads, int dim,
                            int vdim, int rot_dims, float eps, int act, float k_scale, const float* norm_w,
                            int gate_kind, cudaStream_t stream) {
    dim3 grid(n_units, heads, (vdim + 31) / 32);
    if (seq_first_row && (dim == 32 || dim == 64 || dim == 128 || dim == 256)) {
        // a prompt step: chunks of tokens (other key sizes walk the tokens one by one below)
        constexpr int C = kRetChunk;
        size_t chunk_smem = (2 * (size_t)C * (dim + 4) + (size_t)dim * 32 + C * (C + 1) + C * 32 + C + 1) *
                            sizeof(float);
        size_t carry_smem = ((size_t)C * (dim + 4) + (size_t)dim * 32 + seg_len + 1) * sizeof(float);
        dim3 chunk_grid(segments ? n_segments : n_units, heads, (vdim + 31) / 32);
        cudaError_t e = cudaSuccess;
#define NNIS_RET_CHUNK(DR4) \
        do { \
            auto kernel = retention_chunk_kernel<T, DR4>; \
            if (chunk_smem > 48 * 1024) \
                e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)chunk_smem); \
            if (e == cudaSuccess) \
                kernel<<<chunk_grid, 256, chunk_smem, stream>>>((const T*)qkvg, freq, decay, state, seq_slots, \
                                                                seq_first_row, seq_start, seq_count, segments, \
                                                                seg_len, seg_state, o_raw, heads, vdim, rot_dims, act, k_scale); \
            if (e == cudaSuccess && segments) { \
                retention_prefix_kernel<<<dim3(n_units, heads, (dim * vdim + 255) / 256), 256, 0, stream>>>( \
                    seg_state, state, decay, seq_slots, seq_count, seq_first_segment, seg_len, heads, dim * vdim); \
                auto carry = retention_carry_kernel<T, DR4>; \
                if (carry_smem > 48 * 1024) \
                    e = cudaFuncSetAttribute(carry, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)carry_smem); \
                if (e == cudaSuccess) \
                    carry<<<chunk_grid, 256, carry_smem, stream>>>((const T*)qkvg, freq, decay, seg_state, \
                                                                   seq_first_row, seq_start, seq_count, segments, \
                                                                   seg_len, o_raw, heads, vdim, rot_dims, act, k_scale); \
            } \
        } while (0)
        if (dim == 32) NNIS_RET_CHUNK(1);
        else if (dim == 64) NNIS_RET_CHUNK(2);
        else if (dim == 128) NNIS_RET_CHUNK(4);
        else NNIS_RET_CHUNK(8);
#undef NNIS_RET_CHUNK
        if (e != cudaSuccess) return (int)e;
        e = cudaGetLastError();
        if (e != cudaSuccess) return (int)e;
        if (norm_w) {
            retention_gate_joined_kernel<T><<<(unsigned)n_tokens, 256, 0, stream>>>(
                o_raw, (const T*)qkvg, norm_w, token_pos, (T*)out, heads, dim, vdim, eps, gate_kind);
            NNIS_RETURN_LAUNCH();
        }
        long long gate_units = (long long)n_tokens * heads;
        retention_gate_kernel<T><<<(unsigned)((gate_units + 7) / 8), 256, 0, stream>>>(
            o_raw, (const T*)qkvg, token_pos, (T*)out, gate_units, heads, dim, vdim, eps, gate_kind);
        NNIS_RETURN_LAUNCH();
    }
    size_t smem = (2 * (size_t)dim + 256) * sizeof(float);
    cudaError_t le = cudaSuccess;
#define NNIS_RET_CASE(R) \
    le = launch_dependent(retention_scan_kernel<T, R>, grid, 256, smem, stream, (const T*)qkvg, freq, decay, state, \
                          token_pos, token_seq, seq_slots, seq_first_row, seq_start, seq_count, o_raw, heads, dim, \
                          vdim, rot_dims, act, k_scale)
    if (dim <= 32) NNIS_RET_CASE(4);
    else if (dim <= 64) NNIS_RET_CASE(8);
    else if (dim <= 128) NNIS_RET_CASE(16);
    else NNIS_RET_CASE(32);
#undef NNIS_RET_CASE
    if (le != cudaSuccess) return (int)le;
    if (norm_w) {
        le = launch_dependent(retention_gate_joined_kernel<T>, (unsigned)n_tokens, 256, 0, stream,
                              (const float*)o_raw, (const T*)qkvg, norm_w, token_pos, (T*)out, heads, dim, vdim, eps,
                              gate_kind);
        return le == cudaSuccess ? NNIS_OK : (int)le;
    }
    long long units = (long long)n_tokens * heads;
    le = launch_dependent(retention_gate_kernel<T>, (unsigned)((units + 7) / 8), 256, 0, stream,
                          (const float*)o_raw, (const T*)qkvg, token_pos, (T*)out, units, heads, dim, vdim, eps,
                          gate_kind);
    return le == cudaSuccess ? NNIS_OK : (int)le;
}

}  // namespace nnis

using namespace nnis;

// `seq_first_row` null: every row is a sequence of its own bringing one token
// (`n_units` = n_tokens); else `n_units` sequences with their first row, first
// position and token count.  `o_raw`: float32 scratch [n_tokens, heads * vdim].
// `segments` (optional, prompt steps): int32 [n_segments, 2] = (sequence, first token of
// the run among the sequence's tokens of this step), runs of `seg_len` tokens in the order
// of the sequences, with `seq_first_segment` [n_units + 1] and `seg_state` float32
// [n_segments, heads, dim, vdim]: the runs are worked side by side.
// `act` 1: q, k, v through silu; `k_scale`: the keys' multiplier; `norm_w` (float32 [heads * vdim]): one
// norm over the joined heads with this weight instead of a norm per head; `gate_kind` 0 silu, 1 sigmoid.
NNIS_API int nnis_retention(const void* qkvg, const float* freq, const float* decay, float* state,
                            const int* token_pos, const int* token_seq, const int* seq_slots,
                            const int* seq_first_row, const int* seq_start, const int* seq_count,
                            const int* segments, int n_segments, const int* seq_first_segment, int seg_len,
                            float* seg_state, float* o_raw, void* out, int n_tokens, int n_units, int heads, int dim,
                            int vdim, int rot_dims, float eps, int act, float k_scale, const float* norm_w,
                            int gate_kind, int dtype, cudaStream_t stream) {
    if (n_tokens <= 0 || n_units <= 0 || heads <= 0 || dim <= 0 || vdim <= 0 || rot_dims < 0 ||
        (rot_dims & 1) || rot_dims > dim || !(eps > 0.f) || !qkvg || !freq || !decay || !state ||
        !token_pos || !token_seq || !seq_slots || !o_raw || !out)
        return NNIS_ERR_ARGUMENT;
    if (seq_first_row && (!seq_start || !seq_count)) return NNIS_ERR_ARGUMENT;
    // runs side by side: only for prompt steps of key sizes the chunk kernel takes
    if (segments && (!seq_first_row || n_segments <= 0 || !seq_first_segment || !seg_state || seg_len <= 0 ||
                     seg_len % 32 || seg_len > 4096 || !(dim == 32 || dim == 64 || dim == 128 || dim == 256)))
        return NNIS_ERR_ARGUMENT;
    if (dim > 256 || heads > 65535 || (vdim + 31) / 32 > 65535) return NNIS_ERR_UNSUPPORTED;
    if (dtype == NNIS_DTYPE_F32)
        return launch_retention<float>(qkvg, freq, decay, state, token_pos, token_seq, seq_slots,
                                       seq_first_row, seq_start, seq_count, segments, n_segments,
                                       seq_first_segment, seg_len, seg_state, o_raw, out, n_tokens,
                                       n_units, heads, dim, vdim, rot_dims, eps, act, k_scale, norm_w, gate_kind, stream);
    if (dtype == NNIS_DTYPE_BF16)
        return launch_retention<bf16>(qkvg, freq, decay, state, token_pos, token_seq, seq_slots,
                                      seq_first_row, seq_start, seq_count, segments, n_segments,
                                      seq_first_segment, seg_len, seg_state, o_raw, out, n_tokens,
                                      n_units, heads, dim, vdim, rot_dims, eps, act, k_scale, norm_w, gate_kind, stream);
    return NNIS_ERR_UNSUPPORTED;
}
