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
//   delta_prep     a CTA per (token, q or k head or 256 value channels), from the projection's float32 row
//                  [q (G dim) | k (G dim) | v (H vdim) | gate (H vdim) | b (H) | a (H)]:
//                  the causal convolution per channel over the last `taps` inputs (inputs from
//                  before the step come from the state, zeros at a sequence's start) and silu;
//                  every q and k head divided by sqrt(sum of squares + unit_eps), q times
//                  q_scale; beta = sigmoid(b); g = exp(-exp(A_log) * softplus(a + dt_bias)).
//   delta_conv_tail  moves the convolutions' state on by the step's inputs.
//   delta_scan     a CTA per (sequence, head, 32 columns of vdim) walks the step's tokens in order.
//                  A column of S never meets another, so a column is owned by KS (1 to 8) neighbouring
//                  lanes that hold 32 of its values each in registers.  Since
//                  o = g S^T q + u (k . q), the sums S^T k and S^T q are reduced together, one round
//                  of shuffles a token, and k . q is made once a token for all columns.  Tokens come
//                  16 at a time through shared memory.
//   runs           a long prompt is cut into runs (128 tokens) that are walked side by side from
//                  nothing (delta_scan, pass 1, which also yields every run's transition matrix),
//                  put together in order (delta_prefix) and finished by one product a run
//                  (delta_apply): see the kernels.
//   delta_finish   o / rms(o) per head (eps), times a weight per value (shared by the heads),
//                  times silu(gate), rounded once to the operand dtype.
//
// A row whose position is -1 (padding) is skipped everywhere.
#include "async_copy.cuh"
#include "common.cuh"

namespace nnis {

__device__ __forceinline__ float delta_softplus(float x) { return x > 20.f ? x : log1pf(expf(x)); }

// conv_w [conv_cols, taps] (the last column is the current token's); tail [slots, taps - 1, conv_cols].
// A CTA per (`per_cta` tokens, piece): pieces 0 .. 2 G - 1 are the q heads, then the k heads (dim <= 256 channels: a thread
// a channel, then the unit vector); the pieces after them are slabs of 256 value channels; the last piece also
// takes beta and the decay.
__global__ void __launch_bounds__(256)
delta_prep_kernel(const float* __restrict__ a, const float* __restrict__ conv_w, const float* __restrict__ tail,
                  const float* __restrict__ a_log, const float* __restrict__ dt_bias,
                  const int* __restrict__ token_pos, const int* __restrict__ token_seq,
                  const int* __restrict__ seq_slots, const int* __restrict__ seq_first_row,
                  float* __restrict__ qkv, float* __restrict__ beta_g, int n_tokens, int per_cta, int H, int G,
                  int dim, int vdim, int taps, float unit_eps, float q_scale) {
    __shared__ float red[2][8];
    pdl_wait();
    pdl_launch_dependents();
    const int piece = blockIdx.y;
    const int L = taps - 1;
    const int nqk = 2 * G * dim, nv = H * vdim, conv_cols = nqk + nv;
    const int row_len = conv_cols + nv + 2 * H;
    const bool head = piece < 2 * G;
    const int c = head ? piece * dim + (int)threadIdx.x : nqk + (piece - 2 * G) * 256 + (int)threadIdx.x;
    const bool in = head ? (int)threadIdx.x < dim : c < conv_cols;
    for (int j = 0; j < per_cta; ++j) {  // (uniform over the CTA: every thread meets the barrier below)
        const int n = blockIdx.x * per_cta + j;
        if (n >= n_tokens) break;
        if (token_pos[n] < 0) continue;
        const int seq = token_seq[n];
        const int first = seq_first_row ? seq_first_row[seq] : n;
        const float* old = tail + (size_t)seq_slots[seq] * (L > 0 ? L : 1) * conv_cols;
        float y = 0.f;
        if (in) {
            float acc = 0.f;
            for (int t = 0; t < taps; ++t) {
                const int back = L - t;  // tokens before this one
                const float x = n - back >= first ? a[(size_t)(n - back) * row_len + c]
                                                  : old[(size_t)(L - (back - (n - first))) * conv_cols + c];
                acc = fmaf(conv_w[(size_t)c * taps + t], x, acc);
            }
            y = acc / (1.0f + expf(-acc));
        }
        if (head) {
            const float ss = warp_sum(y * y);
            if ((threadIdx.x & 31) == 0) red[j & 1][threadIdx.x >> 5] = ss;
            __syncthreads();  // (two sets of sums in turn: the next token's writers may be ahead of this one's readers)
            float total = 0.f;
#pragma unroll
            for (int w = 0; w < 8; ++w) total += red[j & 1][w];
            if (in) qkv[(size_t)n * conv_cols + c] = y * ((piece < G ? q_scale : 1.0f) / sqrtf(total + unit_eps));
            continue;
        }
        if (in) qkv[(size_t)n * conv_cols + c] = y;
        if (piece + 1 == (int)gridDim.y) {
            const float* row = a + (size_t)n * row_len;
            for (int h = threadIdx.x; h < H; h += 256) {
                beta_g[(size_t)n * 2 * H + h] = 1.0f / (1.0f + expf(-row[conv_cols + nv + h]));
                beta_g[(size_t)n * 2 * H + H + h] =
                    expf(-expf(a_log[h]) * delta_softplus(row[conv_cols + nv + H + h] + dt_bias[h]));
            }
        }
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
constexpr int kDeltaKS = 8;     // lanes that share a column of the state in the kernels after the walk
constexpr int kDeltaNC = 2;     // columns of the state a thread of the walk holds

// KL: state values a thread holds, KS: threads to a column (dim <= KL KS).  qkv float32 [n, 2 G dim + H vdim]; beta_g float32 [n, 2 H].
// PASS 0: a unit is a sequence (or, without the sequences' tables, a row): its tokens of the step in order, from and
//         into the slot's state.
// PASS 1: a unit is a run of `seg_len` tokens (`segments`: sequence, first token), worked from nothing.  The recurrence
//         is linear in the state, S_after = P S_before + S_run with P = prod_t g_t (I - beta_t k_t k_t^T) (later tokens
//         to the left), and every column of the state goes through it alone.  Tiles z < ceil(vdim / 32) hold value
//         columns: they start at zero, leave the run's own outputs in o_raw and S_run in seg_state.  The tiles after
//         them hold `dim` columns that start as the identity and see values of zero: they end as P (seg_trans
//         [runs, H, dim, dim]), and their read-out at token t is P_t^T q_t (q_run [n, H, dim]), with which the part
//         of o_t that comes from before the run is (P_t^T q_t)^T S_before: a product, no second walk (delta_apply).
// The kernels after the walk (delta_prefix, delta_apply) hold a column's values in eight lanes: key channel of
// register r in the eighth `part`.
__device__ __forceinline__ int delta_channel(int r, int part) { return (r >> 2) * 32 + part * 4 + (r & 3); }

// rows of `width` values from global memory into rows of `stride` floats of shared memory, zeros from `width` up to
// W (a constant, so that a thread finds its row and column without a division): the loads of a batch are all issued
// before the first store (shared memory may alias anything, as far as the compiler knows)
template <int W, int NT, typename Src>
__device__ __forceinline__ void delta_stage(float* dst, int stride, int rows, int width, Src src) {
    const int total = rows * W;
    for (int base = 0; base < total; base += NT * 4) {
        float v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int it = base + u * NT + (int)threadIdx.x;
            v[u] = (it < total && it % W < width) ? src(it / W, it % W) : 0.f;
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int it = base + u * NT + (int)threadIdx.x;
            if (it < total) dst[(it / W) * stride + it % W] = v[u];
        }
    }
}

// The walk itself: KS lanes share a column and hold KL = DP / KS of its values each, a CTA of 32 KS threads holds 32
// columns.  Few lanes a column mean few shuffles a token (log2 KS rounds for the two sums) beside its 3 KL multiply-adds,
// so KS is the smallest that leaves a thread 32 values: 2 for keys of 64, 4 for 128, 8 for 256.  Register r of lane
// `part` holds channel (r / 4) 4 KS + 4 part + r % 4: a column's lanes read a token's q and k 16 bytes a load, side by
// side.
template <int KS>
__device__ __forceinline__ int scan_channel(int r, int part) { return (r >> 2) * (4 * KS) + part * 4 + (r & 3); }

template <int KL, int KS, int NC, int PASS>
__global__ void __launch_bounds__(32 * KS)
delta_scan_kernel(const float* __restrict__ qkv, const float* __restrict__ beta_g, float* __restrict__ state,
                  const int* __restrict__ token_pos, const int* __restrict__ token_seq,
                  const int* __restrict__ seq_slots, const int* __restrict__ seq_first_row,
                  const int* __restrict__ seq_count, const int* __restrict__ segments, int seg_len,
                  float* __restrict__ seg_state, float* __restrict__ seg_trans, float* __restrict__ q_run,
                  float* __restrict__ o_raw, int H, int G, int dim, int vdim) {
    constexpr int TT = kDeltaTile, DP = KL * KS, NT = 32 * KS;  // DP: dim rounded up, the tile's row
    constexpr int CW = 32 * NC;                                  // columns of the state a CTA holds
    static_assert(NT >= TT && KL % 4 == 0, "a thread per token of a tile; channels in fours");
    extern __shared__ __align__(16) float smem[];
    float* qs = smem;              // [TT][DP], zero past dim
    float* ks = qs + TT * DP;      // [TT][DP]
    float* vs = ks + TT * DP;      // [TT][CW]
    float* bs = vs + TT * CW;      // [TT] beta
    float* gs = bs + TT;           // [TT] decay
    float* kqs = gs + TT;          // [TT] k . q
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    pdl_wait();
    pdl_launch_dependents();
    const int unit = blockIdx.x, h = blockIdx.y;
    int first, count, slot;
    if (PASS == 1) {
        const int seq = segments[2 * unit], t0 = segments[2 * unit + 1];
        first = seq_first_row[seq] + t0;
        count = min(seg_len, seq_count[seq] - t0);
        slot = 0;
    } else if (seq_first_row) {
        first = seq_first_row[unit];
        count = seq_count[unit];
        slot = seq_slots[unit];
    } else {  // one token per row; a row without a sequence has position -1
        first = unit;
        count = token_pos[unit] < 0 ? 0 : 1;
        slot = seq_slots[token_seq[unit]];
    }
    if (count <= 0) return;
    const int part = tid & (KS - 1);               // which share of the column
    const int cg = tid / KS;                       // which NC of the CTA's columns
    const int value_tiles = (vdim + CW - 1) / CW;
    const bool trans = PASS == 1 && (int)blockIdx.z >= value_tiles;
    const int tile0 = (trans ? (int)blockIdx.z - value_tiles : (int)blockIdx.z) * CW;
    const int col = tile0 + cg * NC;               // the first of the thread's columns of the state
    const int ncols = trans ? dim : vdim;
    const int kv = h / (H / G);
    const int cols = 2 * G * dim + H * vdim;
    float* S = PASS == 0 ? state + (((size_t)slot * H + h) * dim) * vdim
               : trans   ? seg_trans + (((size_t)unit * H + h) * dim) * dim
                         : seg_state + (((size_t)unit * H + h) * dim) * vdim;
    float s[NC][KL];
#pragma unroll
    for (int r = 0; r < KL; ++r) {
        const int d = scan_channel<KS>(r, part);
#pragma unroll
        for (int c = 0; c < NC; ++c) {
            if (PASS == 0) s[c][r] = (col + c < ncols && d < dim) ? S[(size_t)d * vdim + col + c] : 0.f;
            else s[c][r] = (trans && col + c < ncols && d == col + c) ? 1.f : 0.f;
        }
    }
    for (int t0 = 0; t0 < count; t0 += TT) {
        const int cnt = min(TT, count - t0);
        const float* rows = qkv + (size_t)(first + t0) * cols;
        __syncthreads();  // the tile before is read
        delta_stage<DP, NT>(qs, DP, cnt, dim, [&](int i, int d) { return rows[(size_t)i * cols + (size_t)kv * dim + d]; });
        delta_stage<DP, NT>(ks, DP, cnt, dim,
                            [&](int i, int d) { return rows[(size_t)i * cols + (size_t)(G + kv) * dim + d]; });
        delta_stage<CW, NT>(vs, CW, cnt, CW, [&](int i, int c) {
            return (!trans && tile0 + c < vdim) ? rows[(size_t)i * cols + 2 * G * dim + (size_t)h * vdim + tile0 + c] : 0.f;
        });
        if (tid < cnt) {
            bs[tid] = beta_g[(size_t)(first + t0 + tid) * 2 * H + h];
            gs[tid] = beta_g[(size_t)(first + t0 + tid) * 2 * H + H + h];
        }
        __syncthreads();
        for (int i = warp; i < cnt; i += NT / 32) {  // k . q is the same for every column
            float kq = 0.f;
            for (int d = lane; d < DP; d += 32) kq = fmaf(ks[i * DP + d], qs[i * DP + d], kq);
            kq = warp_sum(kq);
            if (lane == 0) kqs[i] = kq;
        }
        __syncthreads();
        for (int i = 0; i < cnt; ++i) {
            const float4* q4 = reinterpret_cast<const float4*>(qs + i * DP + part * 4);
            const float4* k4 = reinterpret_cast<const float4*>(ks + i * DP + part * 4);
            // a thread's NC columns share the token's q and k: one fetch feeds NC sums.  Two chains a sum where a
            // thread has one column (a sum of KL terms is long); NC columns are chains enough
            constexpr int CH = NC == 1 ? 2 : 1;
            float sk[NC][CH], sq[NC][CH];
#pragma unroll
            for (int c = 0; c < NC; ++c)
#pragma unroll
                for (int j = 0; j < CH; ++j) sk[c][j] = sq[c][j] = 0.f;
            float kr[KL];
#pragma unroll
            for (int r4 = 0; r4 < KL / 4; ++r4) {
                const float4 kk = k4[r4 * KS], qq = q4[r4 * KS];
                const float kx[4] = {kk.x, kk.y, kk.z, kk.w}, qx[4] = {qq.x, qq.y, qq.z, qq.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    kr[r4 * 4 + e] = kx[e];
#pragma unroll
                    for (int c = 0; c < NC; ++c) {
                        sk[c][e % CH] = fmaf(s[c][r4 * 4 + e], kx[e], sk[c][e % CH]);
                        sq[c][e % CH] = fmaf(s[c][r4 * 4 + e], qx[e], sq[c][e % CH]);
                    }
                }
            }
            const float g = gs[i], beta = bs[i], kq = kqs[i];
#pragma unroll
            for (int c = 0; c < NC; ++c) {
                float sks = sk[c][0], sqs = sq[c][0];
                if (CH == 2) { sks += sk[c][CH - 1]; sqs += sq[c][CH - 1]; }
#pragma unroll
                for (int o = KS / 2; o > 0; o >>= 1) {
                    sks += __shfl_xor_sync(0xffffffffu, sks, o);
                    sqs += __shfl_xor_sync(0xffffffffu, sqs, o);
                }
                // o = (g S + k u^T)^T q = g S^T q + u (k . q), with S the state before the token
                const float u = beta * (vs[i * CW + cg * NC + c] - g * sks);
#pragma unroll
                for (int r = 0; r < KL; ++r) s[c][r] = fmaf(kr[r], u, g * s[c][r]);
                if (part == 0 && col + c < ncols) {
                    const float o = fmaf(u, kq, g * sqs);
                    if (trans) q_run[((size_t)(first + t0 + i) * H + h) * dim + col + c] = o;
                    else o_raw[((size_t)(first + t0 + i) * H + h) * vdim + col + c] = o;
                }
            }
        }
    }
#pragma unroll
    for (int r = 0; r < KL; ++r) {
        const int d = scan_channel<KS>(r, part);
#pragma unroll
        for (int c = 0; c < NC; ++c)
            if (col + c < ncols && d < dim) S[(size_t)d * ncols + col + c] = s[c][r];
    }
}

// Between the runs' own walk and the product that finishes their outputs: a CTA per (sequence, head, 32 value
// columns) walks the sequence's runs in order.  seg_state[run] (what the run adds) becomes the state before the
// run; the state after it is P_run S_before + S_run, a product with the run's transition taken 32 of its columns at
// a time through shared memory.  A lane owns a column, warp w its rows w, w + 8, ...: a warp reads the transition's
// row 16 bytes a load from ONE address (a broadcast), and the carried column lies along a row of shared memory to be
// read the same way, so 64 multiply-adds take 17 loads of which 16 cost one trip.  The next 32 columns of the
// transition (the next run's first, at a run's end) are fetched into registers while the current ones are
// multiplied.  The slot's state becomes the state after the last run.
constexpr int kDeltaPrefixCols = 32;   // columns of the transition a trip
constexpr int kDeltaApplyNC = 4;       // value columns a thread of the last product holds

template <int KL>
__global__ void __launch_bounds__(256)
delta_prefix_kernel(float* __restrict__ state, const int* __restrict__ seq_slots,
                    const int* __restrict__ seq_first_segment, float* __restrict__ seg_state,
                    const float* __restrict__ seg_trans, int H, int dim, int vdim) {
    constexpr int KS = kDeltaKS, EC = kDeltaPrefixCols, DP = KL * KS;
    constexpr int CS = DP + 4, PS = EC + 4;  // row strides: 16-byte rows, neighbours four banks apart
    static_assert(KS == 8 && EC == 32, "eight warps of 32 lanes: a warp a row of the trip, a lane a column");
    extern __shared__ __align__(16) float smem[];
    float* cs = smem;             // [32][CS]: the carried state, a column of it a row
    float* ps = cs + 32 * CS;     // [DP][PS]: EC columns of the transition, zero past dim
    const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
    pdl_wait();
    pdl_launch_dependents();
    const int seq = blockIdx.x, h = blockIdx.y;
    const int col = blockIdx.z * 32 + lane;
    const bool live = col < vdim;
    float* S = state + (((size_t)seq_slots[seq] * H + h) * dim) * vdim;
    float carry[KL], pre[KL];
#pragma unroll
    for (int r = 0; r < KL; ++r) {
        const int d = w + KS * r;
        carry[r] = (live && d < dim) ? S[(size_t)d * vdim + col] : 0.f;
    }
    // row w + 8 k, column e0 + lane of a run's transition: the thread's share of a trip
    auto fetch = [&](int run, int e0) {
        const float* P = seg_trans + (((size_t)run * H + h) * dim) * dim;
#pragma unroll
        for (int k = 0; k < KL; ++k) {
            const int d = w + KS * k;
            pre[k] = (d < dim && e0 + lane < dim) ? P[(size_t)d * dim + e0 + lane] : 0.f;
        }
    };
    const int first_run = seq_first_segment[seq], last = seq_first_segment[seq + 1];
    if (first_run < last) fetch(first_run, 0);
    for (int run = first_run; run < last; ++run) {
        float* local = seg_state + (((size_t)run * H + h) * dim) * vdim;
        float acc[KL];
#pragma unroll
        for (int r = 0; r < KL; ++r) {
            const int d = w + KS * r;
            acc[r] = (live && d < dim) ? local[(size_t)d * vdim + col] : 0.f;
        }
#pragma unroll
        for (int r = 0; r < KL; ++r) {
            const int d = w + KS * r;
            if (live && d < dim) local[(size_t)d * vdim + col] = carry[r];
            cs[lane * CS + d] = carry[r];
        }
        for (int e0 = 0; e0 < dim; e0 += EC) {
            __syncthreads();  // cs is whole; the trip before is read
#pragma unroll
            for (int k = 0; k < KL; ++k) ps[(w + KS * k) * PS + lane] = pre[k];
            if (e0 + EC < dim) fetch(run, e0 + EC);
            else if (run + 1 < last) fetch(run + 1, 0);
            __syncthreads();
            const float* crow = cs + lane * CS + e0;  // e0 + EC <= DP; past dim both factors are zero
#pragma unroll
            for (int ee = 0; ee < EC; ee += 4) {
                const float4 c = *reinterpret_cast<const float4*>(crow + ee);
#pragma unroll
                for (int r = 0; r < KL; ++r) {
                    const float4 p = *reinterpret_cast<const float4*>(ps + (w + KS * r) * PS + ee);
                    acc[r] = fmaf(p.w, c.w, fmaf(p.z, c.z, fmaf(p.y, c.y, fmaf(p.x, c.x, acc[r]))));
                }
            }
        }
        __syncthreads();  // cs is read before the next run writes it
#pragma unroll
        for (int r = 0; r < KL; ++r) carry[r] = acc[r];
    }
#pragma unroll
    for (int r = 0; r < KL; ++r) {
        const int d = w + KS * r;
        if (live && d < dim) S[(size_t)d * vdim + col] = carry[r];
    }
}

// o_raw[t, h, :] += S_before(run of t)^T q_run[t, h, :]: what the tokens before a run contribute to its outputs.
// A CTA per (run, head, 128 value columns) holds its tile of S_before in registers: eight lanes share four
// neighbouring columns (the scan's layout of channels), so one fetch of a token's q feeds four sums; the sums of 16
// tokens go through shared memory so that a row's values are added to o_raw side by side.
template <int KL>
__global__ void __launch_bounds__(256)
delta_apply_kernel(const float* __restrict__ q_run, const float* __restrict__ seg_state,
                   const int* __restrict__ seq_first_row, const int* __restrict__ seq_count,
                   const int* __restrict__ segments, int seg_len, float* __restrict__ o_raw, int H, int dim,
                   int vdim) {
    constexpr int KS = kDeltaKS, TT = kDeltaTile, DP = KL * KS, NC = kDeltaApplyNC, CW = 32 * NC;
    extern __shared__ __align__(16) float smem[];
    float* qs = smem;            // [TT][DP], zero past dim
    float* os = qs + TT * DP;    // [TT][CW]
    const int tid = threadIdx.x, part = tid & (KS - 1), cg = tid >> 3;
    for (int i = tid; i < TT * DP; i += 256) qs[i] = 0.f;
    pdl_wait();
    pdl_launch_dependents();
    const int unit = blockIdx.x, h = blockIdx.y;
    const int seq = segments[2 * unit], t_first = segments[2 * unit + 1];
    const int first = seq_first_row[seq] + t_first;
    const int count = min(seg_len, seq_count[seq] - t_first);
    if (count <= 0) return;
    const int tile0 = blockIdx.z * CW;
    const int col = tile0 + cg * NC;  // the first of the thread's columns
    const float* S = seg_state + (((size_t)unit * H + h) * dim) * vdim;
    float s[NC][KL];
#pragma unroll
    for (int r = 0; r < KL; ++r) {
        const int d = delta_channel(r, part);
#pragma unroll
        for (int c = 0; c < NC; ++c) s[c][r] = (col + c < vdim && d < dim) ? S[(size_t)d * vdim + col + c] : 0.f;
    }
    for (int t0 = 0; t0 < count; t0 += TT) {
        const int cnt = min(TT, count - t0);
        __syncthreads();
        delta_stage<DP, 256>(qs, DP, cnt, dim, [&](int i, int d) { return q_run[((size_t)(first + t0 + i) * H + h) * dim + d]; });
        __syncthreads();
#pragma unroll 2
        for (int i = 0; i < cnt; ++i) {
            const float4* q4 = reinterpret_cast<const float4*>(qs + i * DP + part * 4);
            float acc[NC];
#pragma unroll
            for (int c = 0; c < NC; ++c) acc[c] = 0.f;
#pragma unroll
            for (int r4 = 0; r4 < KL / 4; ++r4) {
                const float4 qq = q4[r4 * 8];
#pragma unroll
                for (int c = 0; c < NC; ++c) {
                    acc[c] = fmaf(s[c][r4 * 4], qq.x, acc[c]);
                    acc[c] = fmaf(s[c][r4 * 4 + 1], qq.y, acc[c]);
                    acc[c] = fmaf(s[c][r4 * 4 + 2], qq.z, acc[c]);
                    acc[c] = fmaf(s[c][r4 * 4 + 3], qq.w, acc[c]);
                }
            }
#pragma unroll
            for (int c = 0; c < NC; ++c) {
#pragma unroll
                for (int o = KS / 2; o > 0; o >>= 1) acc[c] += __shfl_xor_sync(0xffffffffu, acc[c], o);
            }
            if (part == 0) *reinterpret_cast<float4*>(os + i * CW + cg * NC) = make_float4(acc[0], acc[1], acc[2], acc[3]);
        }
        __syncthreads();
        for (int it = tid; it < cnt * CW; it += 256) {
            const int i = it / CW, c = tile0 + it % CW;
            if (c < vdim) o_raw[((size_t)(first + t0 + i) * H + h) * vdim + c] += os[it];
        }
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
    if (dim > 256 || taps > 64 || 2 * G + (H * vdim + 255) / 256 > 65535) return NNIS_ERR_UNSUPPORTED;
    const int per_cta = n_tokens > 256 ? 8 : 1;  // prompt steps: fewer, longer CTAs
    const dim3 pieces((n_tokens + per_cta - 1) / per_cta, 2 * G + (H * vdim + 255) / 256);
    cudaError_t e = launch_dependent(delta_prep_kernel, pieces, 256, 0, stream, a, conv_w,
                                     (const float*)tail, a_log, dt_bias, token_pos, token_seq, seq_slots,
                                     seq_first_row, qkv, beta_g, n_tokens, per_cta, H, G, dim, vdim, taps, unit_eps,
                                     q_scale);
    if (e != cudaSuccess) return (int)e;
    if (taps > 1) {
        const int conv_cols = 2 * G * dim + H * vdim;
        dim3 grid(n_units, (conv_cols + 255) / 256);
        e = launch_dependent(delta_conv_tail_kernel, grid, 256, 0, stream, a, tail, token_pos, token_seq, seq_slots,
                             seq_first_row, seq_count, conv_cols, conv_cols + H * vdim + 2 * H, taps);
    }
    return e == cudaSuccess ? NNIS_OK : (int)e;
}

namespace nnis {

template <int KL, int SKL, int SKS, int SNC>
static cudaError_t delta_passes(const float* qkv, const float* beta_g, float* state, const int* token_pos,
                                const int* token_seq, const int* seq_slots, const int* seq_first_row,
                                const int* seq_count, const int* segments, int n_segments,
                                const int* seq_first_segment, int seg_len, float* seg_state, float* seg_trans,
                                float* q_run, float* o_raw, int n_units, int H, int G, int dim, int vdim,
                                cudaStream_t stream) {
    constexpr int CW = 32 * SNC;               // the walk's own tiles
    const int walk_tiles = (vdim + CW - 1) / CW;
    const size_t smem = ((size_t)2 * kDeltaTile * SKL * SKS + kDeltaTile * CW + 3 * kDeltaTile) * sizeof(float);
    if (!segments)
        return launch_dependent(delta_scan_kernel<SKL, SKS, SNC, 0>, dim3(n_units, H, walk_tiles), 32 * SKS, smem, stream, qkv,
                                beta_g, state, token_pos, token_seq, seq_slots, seq_first_row, seq_count, segments,
                                seg_len, seg_state, seg_trans, q_run, o_raw, H, G, dim, vdim);
    cudaError_t e = launch_dependent(delta_scan_kernel<SKL, SKS, SNC, 1>, dim3(n_segments, H, walk_tiles + (dim + CW - 1) / CW),
                                     32 * SKS, smem, stream, qkv, beta_g, state, token_pos, token_seq, seq_slots,
                                     seq_first_row, seq_count, segments, seg_len, seg_state, seg_trans, q_run, o_raw,
                                     H, G, dim, vdim);
    if (e != cudaSuccess) return e;
    const size_t prefix_smem = ((size_t)32 * (KL * kDeltaKS + 4) +
                                (size_t)KL * kDeltaKS * (kDeltaPrefixCols + 4)) * sizeof(float);
    if (prefix_smem > 48 * 1024) {
        e = cudaFuncSetAttribute(delta_prefix_kernel<KL>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)prefix_smem);
        if (e != cudaSuccess) return e;
    }
    e = launch_dependent(delta_prefix_kernel<KL>, dim3(n_units, H, (vdim + 31) / 32), 256, prefix_smem, stream, state,
                         seq_slots, seq_first_segment, seg_state, (const float*)seg_trans, H, dim, vdim);
    if (e != cudaSuccess) return e;
    constexpr int apply_cols = 32 * kDeltaApplyNC;
    return launch_dependent(delta_apply_kernel<KL>, dim3(n_segments, H, (vdim + apply_cols - 1) / apply_cols), 256,
                            (size_t)kDeltaTile * (KL * kDeltaKS + apply_cols) * sizeof(float), stream,
                            (const float*)q_run, (const float*)seg_state, seq_first_row, seq_count, segments, seg_len,
                            o_raw, H, dim, vdim);
}

}  // namespace nnis

// state float32 [slots, H, dim, vdim]; o_raw float32 [n, H vdim].  `units`: sequences of the step (with
// seq_first_row) or rows.  With `segments` (int32 [n_segments, 2] = (sequence, first token of the run), runs of
// seg_len tokens), seq_first_segment [sequences + 1] and scratch seg_state float32 [n_segments, H, dim, vdim],
// seg_trans float32 [n_segments, H, dim, dim] and q_run float32 [n, H, dim] the runs are worked side by side.
NNIS_API int nnis_delta_scan(const float* qkv, const float* beta_g, float* state, const int* token_pos,
                             const int* token_seq, const int* seq_slots, const int* seq_first_row,
                             const int* seq_count, const int* segments, int n_segments,
                             const int* seq_first_segment, int seg_len, float* seg_state, float* seg_trans,
                             float* q_run, float* o_raw, int n_units, int H, int G, int dim, int vdim,
                             cudaStream_t stream) {
    if (n_units <= 0 || H <= 0 || G <= 0 || H % G || dim <= 0 || vdim <= 0 || !qkv || !beta_g || !state ||
        !token_pos || !token_seq || !seq_slots || !o_raw)
        return NNIS_ERR_ARGUMENT;
    if (seq_first_row && !seq_count) return NNIS_ERR_ARGUMENT;
    if (segments && (!seq_first_row || !seq_first_segment || n_segments <= 0 || seg_len <= 0 || !seg_state ||
                     !seg_trans || !q_run))
        return NNIS_ERR_ARGUMENT;
    if (dim > 256 || H > 65535 || (vdim + 31) / 32 > 65535) return NNIS_ERR_UNSUPPORTED;
    cudaError_t e;
#define NNIS_DELTA_CASE(KL, SKL, SKS, SNC) \
    e = delta_passes<KL, SKL, SKS, SNC>(qkv, beta_g, state, token_pos, token_seq, seq_slots, seq_first_row, seq_count, segments, \
                         n_segments, seq_first_segment, seg_len, seg_state, seg_trans, q_run, o_raw, n_units, H, G, \
                         dim, vdim, stream)
    if (dim <= 32) NNIS_DELTA_CASE(4, 32, 1, kDeltaNC);
    else if (dim <= 64) NNIS_DELTA_CASE(8, 32, 2, kDeltaNC);
    else if (dim <= 128) NNIS_DELTA_CASE(16, 32, 4, kDeltaNC);
    else NNIS_DELTA_CASE(32, 32, 8, kDeltaNC);
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
