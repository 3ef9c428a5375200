// Gated delta rule: a recurrent mixer whose state is corrected toward each new value
// instead of only added to.  Per head, with unit vectors q and k (q also times `q_scale`), a
// write strength beta in (0, 1) and a decay g in (0, 1) per token:
//
//     S <- g S        u = beta (v - S^T k)        S <- S + k u^T        o = S^T q
//
// S [dim, vdim] is float32 in a per-sequence state area, starts at zero and is carried from
// step to step; so are the last taps - 1 inputs of the short convolutions in front of q, k
// and v (float32 [taps - 1, channels], oldest first).  Everything after the projections is
// float32 in every dtype.
//
//   delta_prep     a CTA per token, from the projection's float32 row
//                  [q (G dim) | k (G dim) | v (H vdim) | gate (H vdim) | b (H) | a (H)]:
//                  the causal convolution per channel over the last `taps` inputs (inputs from
//                  before the step come from the state, zeros at a sequence's start) and silu;
//                  every q and k head divided by sqrt(sum of squares + unit_eps), q times
//                  q_scale; beta = sigmoid(b); g = exp(-exp(A_log) * softplus(a + dt_bias)).
//   delta_conv_tail  moves the convolutions' state on by the step's inputs.
//   delta_scan     a CTA per (sequence, head, 32 columns of vdim) walks the step's tokens in order.
//                  A column of S never meets another, so a column is owned by KS = 8 neighbouring
//                  lanes that hold dim / 8 of its values each in registers.  Since
//                  o = g S^T q + u (k . q), the three sums S^T k, S^T q and k . q are reduced
//                  together: one round of shuffles a token.  Tokens come 16 at a time through
//                  shared memory.
//   delta_finish   o / rms(o) per head (eps), times a weight per value (shared by the heads),
//                  times silu(gate), rounded once to the operand dtype.
//
// A row whose position is -1 (padding) is skipped everywhere.
#include "async_copy.cuh"
#include "common.cuh"

namespace nnis {

__device__ __forceinline__ float delta_softplus(float x) { return x > 20.f ? x : log1pf(expf(x)); }

// conv_w [conv_cols, taps] (the last column is the current token's); tail [slots, taps - 1, conv_cols]
__global__ void __launch_bounds__(256)
delta_prep_kernel(const float* __restrict__ a, const float* __restrict__ conv_w, const float* __restrict__ tail,
                  const float* __restrict__ a_log, const float* __restrict__ dt_bias,
                  const int* __restrict__ token_pos, const int* __restrict__ token_seq,
                  const int* __restrict__ seq_slots, const int* __restrict__ seq_first_row,
                  float* __restrict__ qkv, float* __restrict__ beta_g, int H, int G, int dim, int vdim, int taps,
                  float unit_eps, float q_scale) {
    extern __shared__ float conv_out[];  // [2 G dim] q and k after convolution and silu
    pdl_wait();
    pdl_launch_dependents();
    const int n = blockIdx.x;
    if (token_pos[n] < 0) return;
    const int seq = token_seq[n];
    const int slot = seq_slots[seq];
    const int first = seq_first_row ? seq_first_row[seq] : n;
    const int L = taps - 1;
    const int nqk = 2 * G * dim, nv = H * vdim, conv_cols = nqk + nv;
    const int row_len = conv_cols + nv + 2 * H;
    const float* old = tail + (size_t)slot * (L > 0 ? L : 1) * conv_cols;
    for (int c = threadIdx.x; c < conv_cols; c += 256) {
        float acc = 0.f;
        for (int j = 0; j < taps; ++j) {
            const int back = L - j;  // tokens before this one
            const float in = n - back >= first ? a[(size_t)(n - back) * row_len + c]
                                               : old[(size_t)(L - (back - (n - first))) * conv_cols + c];
            acc = fmaf(conv_w[(size_t)c * taps + j], in, acc);
        }
        const float y = acc / (1.0f + expf(-acc));
        if (c < nqk) conv_out[c] = y;
        else qkv[(size_t)n * conv_cols + c] = y;
    }
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int hh = warp; hh < 2 * G; hh += 8) {  // q heads, then k heads
        const float* src = conv_out + (size_t)hh * dim;
        float ss = 0.f;
        for (int i = lane; i < dim; i += 32) ss = fmaf(src[i], src[i], ss);
        const float inv = (hh < G ? q_scale : 1.0f) / sqrtf(warp_sum(ss) + unit_eps);
        float* dst = qkv + (size_t)n * conv_cols + (size_t)hh * dim;
        for (int i = lane; i < dim; i += 32) dst[i] = src[i] * inv;
    }
    const float* row = a + (size_t)n * row_len;
    for (int h = threadIdx.x; h < H; h += 256) {
        beta_g[(size_t)n * 2 * H + h] = 1.0f / (1.0f + expf(-row[conv_cols + nv + h]));
        beta_g[(size_t)n * 2 * H + H + h] =
            expf(-expf(a_log[h]) * delta_softplus(row[conv_cols + nv + H + h] + dt_bias[h]));
    }
}

// new tail[j] = the input `L - j` tokens before the end of the sequence's step; inputs from before
// the step are the old tail's.  A thread per channel walks j upwards: it reads ahead of what it writes.
__global__ void __launch_bounds__(256)
delta_conv_tail_kernel(const float* __restrict__ a, float* __restrict__ tail, const int* __restrict__ token_pos,
                       const int* __restrict__ token_seq, const int* __restrict__ seq_slots,
                       const int* __restrict__ seq_first_row, const int* __restrict__ seq_count, int conv_cols,
                       int row_len, int taps) {
    pdl_wait();
    pdl_launch_dependents();
    const int unit = blockIdx.x;
    int first, count, slot;
    if (seq_first_row) {
        first = seq_first_row[unit];
        count = seq_count[unit];
        slot = seq_slots[unit];
    } else {
        first = unit;
        count = token_pos[unit] < 0 ? 0 : 1;
        slot = seq_slots[token_seq[unit]];
    }
    const int L = taps - 1;
    if (count <= 0 || L <= 0) return;
    float* t = tail + (size_t)slot * L * conv_cols;
    for (int c = blockIdx.y * 256 + threadIdx.x; c < conv_cols; c += 256 * gridDim.y)
        for (int j = 0; j < L; ++j) {
            const int idx = count - L + j;  // among the step's tokens of the sequence
            t[(size_t)j * conv_cols + c] = idx >= 0 ? a[(size_t)(first + idx) * row_len + c]
                                                    : t[(size_t)(j + count) * conv_cols + c];
        }
}

constexpr int kDeltaTile = 16;  // tokens a trip through shared memory
constexpr int kDeltaKS = 8;     // lanes that share a column of the state

// KL: state values a thread holds (dim <= 8 KL).  qkv float32 [n, 2 G dim + H vdim]; beta_g float32 [n, 2 H].
template <int KL>
__global__ void __launch_bounds__(256)
delta_scan_kernel(const float* __restrict__ qkv, const float* __restrict__ beta_g, float* __restrict__ state,
                  const int* __restrict__ token_pos, const int* __restrict__ token_seq,
                  const int* __restrict__ seq_slots, const int* __restrict__ seq_first_row,
                  const int* __restrict__ seq_count, float* __restrict__ o_raw, int H, int G, int dim, int vdim) {
    constexpr int KS = kDeltaKS, TT = kDeltaTile;
    extern __shared__ __align__(16) float smem[];
    float* qs = smem;              // [TT][dim]
    float* ks = qs + TT * dim;     // [TT][dim]
    float* vs = ks + TT * dim;     // [TT][32]
    float* bs = vs + TT * 32;      // [TT] beta
    float* gs = bs + TT;           // [TT] decay
    pdl_wait();
    pdl_launch_dependents();
    const int unit = blockIdx.x, h = blockIdx.y;
    int first, count, slot;
    if (seq_first_row) {
        first = seq_first_row[unit];
        count = seq_count[unit];
        slot = seq_slots[unit];
    } else {  // one token per row; a row without a sequence has position -1
        first = unit;
        count = token_pos[unit] < 0 ? 0 : 1;
        slot = seq_slots[token_seq[unit]];
    }
    if (count <= 0) return;
    const int tid = threadIdx.x;
    const int part = tid & (KS - 1);               // which eighth of the column
    const int col = blockIdx.z * 32 + (tid >> 3);  // the column of the state
    const bool live = col < vdim;
    const int kv = h / (H / G);
    const int cols = 2 * G * dim + H * vdim;
    float* S = state + (((size_t)slot * H + h) * dim) * vdim;
    float s[KL];
#pragma unroll
    for (int i = 0; i < KL; ++i) {
        const int d = i * KS + part;
        s[i] = (live && d < dim) ? S[(size_t)d * vdim + col] : 0.f;
    }
    for (int t0 = 0; t0 < count; t0 += TT) {
        const int cnt = min(TT, count - t0);
        __syncthreads();  // the tile before is read
        for (int it = tid; it < cnt * dim; it += 256) {
            const int i = it / dim, d = it - i * dim;
            const float* row = qkv + (size_t)(first + t0 + i) * cols;
            qs[it] = row[(size_t)kv * dim + d];
            ks[it] = row[(size_t)(G + kv) * dim + d];
        }
        for (int it = tid; it < cnt * 32; it += 256) {
            const int i = it >> 5, c = blockIdx.z * 32 + (it & 31);
            vs[it] = c < vdim ? qkv[(size_t)(first + t0 + i) * cols + 2 * G * dim + (size_t)h * vdim + c] : 0.f;
        }
        if (tid < cnt) {
            bs[tid] = beta_g[(size_t)(first + t0 + tid) * 2 * H + h];
            gs[tid] = beta_g[(size_t)(first + t0 + tid) * 2 * H + H + h];
        }
        __syncthreads();
        for (int i = 0; i < cnt; ++i) {
            const float* q = qs + i * dim;
            const float* k = ks + i * dim;
            float sk = 0.f, sq = 0.f, kq = 0.f;
            float kr[KL];
#pragma unroll
            for (int r = 0; r < KL; ++r) {
                const int d = r * KS + part;
                const float kd = d < dim ? k[d] : 0.f, qd = d < dim ? q[d] : 0.f;
                kr[r] = kd;
                sk = fmaf(s[r], kd, sk);
                sq = fmaf(s[r], qd, sq);
                kq = fmaf(kd, qd, kq);
            }
#pragma unroll
            for (int o = KS / 2; o > 0; o >>= 1) {
                sk += __shfl_xor_sync(0xffffffffu, sk, o);
                sq += __shfl_xor_sync(0xffffffffu, sq, o);
                kq += __shfl_xor_sync(0xffffffffu, kq, o);
            }
            const float g = gs[i];
            const float u = bs[i] * (vs[i * 32 + (tid >> 3)] - g * sk);
#pragma unroll
            for (int r = 0; r < KL; ++r) s[r] = fmaf(kr[r], u, g * s[r]);
            if (part == 0 && live)
                o_raw[((size_t)(first + t0 + i) * H + h) * vdim + col] = fmaf(u, kq, g * sq);
        }
    }
#pragma unroll
    for (int i = 0; i < KL; ++i) {
        const int d = i * KS + part;
        if (live && d < dim) S[(size_t)d * vdim + col] = s[i];
    }
}

// out[n, h, :] = o[n, h, :] / sqrt(mean(o[n, h, :]^2) + eps) * w * silu(gate[n, h, :]); a warp per
// (token, head); `gate` are float32 rows of `gate_stride` values, the head's gate at gate_off + h vdim
template <typename T>
__global__ void __launch_bounds__(256)
delta_finish_kernel(const float* __restrict__ o_raw, const float* __restrict__ gate_rows, int gate_stride,
                    int gate_off, const float* __restrict__ w, const int* __restrict__ token_pos,
                    T* __restrict__ out, long long n_units, int heads, int vdim, float eps) {
    pdl_wait();
    pdl_launch_dependents();
    long long unit = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (unit >= n_units) return;
    const int lane = threadIdx.x & 31;
    const long long n = unit / heads;
    const int h = (int)(unit - n * heads);
    T* dst = out + (size_t)unit * vdim;
    if (token_pos[n] < 0) {
        for (int i = lane; i < vdim; i += 32) dst[i] = from_float<T>(0.f);
        return;
    }
    const float* o = o_raw + (size_t)unit * vdim;
    const float* gate = gate_rows + (size_t)n * gate_stride + gate_off + (size_t)h * vdim;
    float ss = 0.f;
    for (int i = lane; i < vdim; i += 32) ss = fmaf(o[i], o[i], ss);
    const float s = 1.0f / sqrtf(warp_sum(ss) / (float)vdim + eps);
    for (int i = lane; i < vdim; i += 32) {
        const float z = gate[i];
        dst[i] = from_float<T>((o[i] * s) * w[i] * (z / (1.0f + expf(-z))));
    }
}

}  // namespace nnis

using namespace nnis;

// a: float32 [n, 2 G dim + 2 H vdim + 2 H] (see the top); conv_w float32 [2 G dim + H vdim, taps];
// tail float32 [slots, max(taps - 1, 1), 2 G dim + H vdim]; a_log, dt_bias float32 [H];
// qkv float32 [n, 2 G dim + H vdim] and beta_g float32 [n, 2 H] receive what the recurrence reads.
// `seq_first_row` null: every row is a sequence of its own bringing one token.
NNIS_API int nnis_delta_prep(const float* a, const float* conv_w, float* tail, const float* a_log,
                             const float* dt_bias, const int* token_pos, const int* token_seq,
                             const int* seq_slots, const int* seq_first_row, const int* seq_count, float* qkv,
                             float* beta_g, int n_tokens, int n_units, int H, int G, int dim, int vdim, int taps,
                             float unit_eps, float q_scale, cudaStream_t stream) {
    if (n_tokens <= 0 || n_units <= 0 || H <= 0 || G <= 0 || H % G || dim <= 0 || vdim <= 0 || taps < 1 ||
        !(unit_eps > 0.f) || !a || !conv_w || !tail || !a_log || !dt_bias || !token_pos || !token_seq ||
        !seq_slots || !qkv || !beta_g)
        return NNIS_ERR_ARGUMENT;
    if (seq_first_row && !seq_count) return NNIS_ERR_ARGUMENT;
    const size_t smem = (size_t)2 * G * dim * sizeof(float);
    if (smem > 48 * 1024 || taps > 64) return NNIS_ERR_UNSUPPORTED;
    cudaError_t e = launch_dependent(delta_prep_kernel, (unsigned)n_tokens, 256, smem, stream, a, conv_w,
                                     (const float*)tail, a_log, dt_bias, token_pos, token_seq, seq_slots,
                                     seq_first_row, qkv, beta_g, H, G, dim, vdim, taps, unit_eps, q_scale);
    if (e != cudaSuccess) return (int)e;
    if (taps > 1) {
        const int conv_cols = 2 * G * dim + H * vdim;
        dim3 grid(n_units, (conv_cols + 255) / 256);
        e = launch_dependent(delta_conv_tail_kernel, grid, 256, 0, stream, a, tail, token_pos, token_seq, seq_slots,
                             seq_first_row, seq_count, conv_cols, conv_cols + H * vdim + 2 * H, taps);
    }
    return e == cudaSuccess ? NNIS_OK : (int)e;
}

// state float32 [slots, H, dim, vdim]; o_raw float32 [n, H vdim]
NNIS_API int nnis_delta_scan(const float* qkv, const float* beta_g, float* state, const int* token_pos,
                             const int* token_seq, const int* seq_slots, const int* seq_first_row,
                             const int* seq_count, float* o_raw, int n_units, int H, int G, int dim, int vdim,
                             cudaStream_t stream) {
    if (n_units <= 0 || H <= 0 || G <= 0 || H % G || dim <= 0 || vdim <= 0 || !qkv || !beta_g || !state ||
        !token_pos || !token_seq || !seq_slots || !o_raw)
        return NNIS_ERR_ARGUMENT;
    if (seq_first_row && !seq_count) return NNIS_ERR_ARGUMENT;
    if (dim > 256 || H > 65535 || (vdim + 31) / 32 > 65535) return NNIS_ERR_UNSUPPORTED;
    dim3 grid(n_units, H, (vdim + 31) / 32);
    const size_t smem = ((size_t)2 * kDeltaTile * dim + kDeltaTile * 32 + 2 * kDeltaTile) * sizeof(float);
    cudaError_t e;
#define NNIS_DELTA_CASE(KL) \
    e = launch_dependent(delta_scan_kernel<KL>, grid, 256, smem, stream, qkv, beta_g, state, token_pos, token_seq, \
                         seq_slots, seq_first_row, seq_count, o_raw, H, G, dim, vdim)
    if (dim <= 32) NNIS_DELTA_CASE(4);
    else if (dim <= 64) NNIS_DELTA_CASE(8);
    else if (dim <= 128) NNIS_DELTA_CASE(16);
    else NNIS_DELTA_CASE(32);
#undef NNIS_DELTA_CASE
    return e == cudaSuccess ? NNIS_OK : (int)e;
}

// o_raw float32 [n, heads * vdim]; gate_rows float32 [n, gate_stride]; w float32 [vdim]; out [n, heads * vdim]
NNIS_API int nnis_delta_finish(const float* o_raw, const float* gate_rows, int gate_stride, int gate_off,
                               const float* w, const int* token_pos, void* out, int n_tokens, int heads, int vdim,
                               float eps, int dtype, cudaStream_t stream) {
    if (n_tokens <= 0 || heads <= 0 || vdim <= 0 || !(eps > 0.f) || !o_raw || !gate_rows || !w || !token_pos || !out)
        return NNIS_ERR_ARGUMENT;
    const long long units = (long long)n_tokens * heads;
    cudaError_t e;
    if (dtype == NNIS_DTYPE_F32)
        e = launch_dependent(delta_finish_kernel<float>, (unsigned)((units + 7) / 8), 256, 0, stream, o_raw, gate_rows,
                             gate_stride, gate_off, w, token_pos, (float*)out, units, heads, vdim, eps);
    else if (dtype == NNIS_DTYPE_BF16)
        e = launch_dependent(delta_finish_kernel<bf16>, (unsigned)((units + 7) / 8), 256, 0, stream, o_raw, gate_rows,
                             gate_stride, gate_off, w, token_pos, (bf16*)out, units, heads, vdim, eps);
    else
        return NNIS_ERR_UNSUPPORTED;
    return e == cudaSuccess ? NNIS_OK : (int)e;
}
