// Mixture of experts, token by token: a router picks `top` of `experts` small
// feed-forward layers W_down act(W_up h), act = relu^2, and the token's output is
// the sum of theirs weighted by a softmax over the chosen logits only.
//
//   moe_route   logits z = W_r h + b in float32 (a CTA per token, a warp per expert), the `top` largest
//               (ties to the lower index), softmax over those -> ids, weights
//   moe_up      act[n, s, :] = relu(W_up[id[n, s]] h_n)^2: a warp per output feature
//   moe_down    residual[n, :] += sum_s weight[n, s] W_down[id[n, s]] act[n, s, :], the
//               chosen experts added in the router's order (the same bits every time)
//
// A second form serves routers whose scores are sigmoid(z), used as they are (not
// renormalised) and applied to the expert's INPUT, with gated experts
// W_down (silu(W_gate x) * (W_up x)), x = score * h:
//
//   moe_route      with `sigmoid_scores`: the same choice, weights = sigmoid of the chosen logits
//   moe_up_gated   act[n, s, :] = silu(w g) * (w u) with g = W_gate h, u = W_up h and w the score:
//                  the score multiplies both float32 sums, which is the product with w * h
//   moe_down       with no weights: the chosen experts' outputs are added as they are
//
// A third form serves routers that score ALL their outputs with one softmax and choose by those
// scores plus a correction per output, group by group, and whose last outputs stand for experts
// that hand their input on unchanged:
//
//   moe_route_choice  s = softmax(z) over all `outputs`; choice c = s + correction; the outputs form
//                     `groups` equal runs of neighbours, a run's score is its largest c, and only the
//                     `keep` best runs can be chosen (the others' c counts as minus infinity); the `top`
//                     largest c (ties to the lower index) are chosen and weighed by their s as it is.
//                     Outputs from `experts` on have no matrices: their id is written as -1 and their
//                     weights are added up in `pass_weight[n]`
//   moe_up_gated      with no weights: act = silu(g) * u; a pair whose id is negative is skipped
//   moe_down          with weights on the outputs, skipping negative ids, plus pass_weight[n] * h[n]
//
// Expert weights are stacked: W_up [experts, ff, width] (gated: [experts, 2 ff, width], row 2f the
// gate's and row 2f + 1 the up-projection's of feature f), W_down [experts, width, ff].
// A row whose position is -1 (padding) is skipped everywhere.
#include <float.h>

#include "async_copy.cuh"
#include "common.cuh"

namespace nnis {

// sum over a warp's share of two rows' product: 16-byte loads where the rows are bfloat16,
// a multiple of eight long and 16-byte aligned, else element by element
template <typename T>
__device__ __forceinline__ float warp_row_dot(const T* __restrict__ a, const T* __restrict__ b, int len, int lane) {
    float acc = 0.f;
    if (sizeof(T) == 2 && len % 8 == 0 && (((uintptr_t)a | (uintptr_t)b) & 15) == 0) {
        const uint4* a4 = reinterpret_cast<const uint4*>(a);
        const uint4* b4 = reinterpret_cast<const uint4*>(b);
        for (int i = lane; i < len / 8; i += 32) {
            uint4 x = a4[i], y = b4[i];
            const uint32_t xs[4] = {x.x, x.y, x.z, x.w}, ys[4] = {y.x, y.y, y.z, y.w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                acc = fmaf(__uint_as_float(xs[k] << 16), __uint_as_float(ys[k] << 16), acc);
                acc = fmaf(__uint_as_float(xs[k] & 0xffff0000u), __uint_as_float(ys[k] & 0xffff0000u), acc);
            }
        }
    } else {
        for (int i = lane; i < len; i += 32) acc = fmaf(to_float(a[i]), to_float(b[i]), acc);
    }
    return warp_sum(acc);
}

template <typename T>
__global__ void __launch_bounds__(256)
moe_route_kernel(const T* __restrict__ h, const float* __restrict__ wr, const float* __restrict__ br,
                 const int* __restrict__ token_pos, int* __restrict__ ids,
                 float* __restrict__ weights, int n_tokens, int width, int experts, int top,
                 int sigmoid_scores) {
    extern __shared__ float z[];  // [experts]
    pdl_wait();
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int n = blockIdx.x;
    int* id = ids + (size_t)n * top;
    float* wt = weights + (size_t)n * top;
    if (token_pos[n] < 0) {
        for (int s = threadIdx.x; s < top; s += 256) {
            id[s] = 0;
            wt[s] = 0.f;
        }
        return;
    }
    const T* x = h + (size_t)n * width;
    const bool by_four = (width & 3) == 0;  // rows of the router and of x start on 16- and 8-byte borders
    for (int e = warp; e < experts; e += 8) {  // a warp per expert, eight at a time
        const float* w = wr + (size_t)e * width;
        float acc = 0.f;
        if (by_four) {  // several loads in flight per lane: the dot products are latency, not arithmetic
#pragma unroll 4
            for (int i = lane * 4; i < width; i += 128) {
                float4 wv = load4(w + i), xv = load4(x + i);
                acc = fmaf(wv.x, xv.x, acc);
                acc = fmaf(wv.y, xv.y, acc);
                acc = fmaf(wv.z, xv.z, acc);
                acc = fmaf(wv.w, xv.w, acc);
            }
        } else {
            for (int i = lane; i < width; i += 32) acc = fmaf(w[i], to_float(x[i]), acc);
        }
        acc = warp_sum(acc);
        if (lane == 0) z[e] = acc + (br ? br[e] : 0.f);
    }
    __syncthreads();
    if (warp != 0) return;
    // the `top` largest, one after another; the lanes of one warp share the search
    float first = 0.f, total = 0.f;
    for (int s = 0; s < top; ++s) {
        float best = -FLT_MAX;
        int arg = 0x7fffffff;
        for (int e = lane; e < experts; e += 32) {
            float v = z[e];
            if (v > best) {  // (ascending e: the lower index wins a tie)
                best = v;
                arg = e;
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            float ob = __shfl_xor_sync(0xffffffffu, best, o);
            int oa = __shfl_xor_sync(0xffffffffu, arg, o);
            if (ob > best || (ob == best && oa < arg)) {
                best = ob;
                arg = oa;
            }
        }
        if (s == 0) first = best;
        float p = sigmoid_scores ? 1.0f / (1.0f + expf(-best)) : expf(best - first);
        total += p;
        if (lane == 0) {
            id[s] = arg;
            wt[s] = p;
            z[arg] = -FLT_MAX;
        }
        __syncwarp();
    }
    if (sigmoid_scores) return;  // (used as they are)
    float inv = 1.0f / total;
    __syncwarp();
    for (int s = lane; s < top; s += 32) wt[s] *= inv;
}

// A CTA takes TOK tokens.  Shared memory, per token: [outputs] scores, [outputs] choices, [groups] the
// runs' best.  The logits: with one token a warp takes four outputs at a time (their rows' loads are in
// flight together); with several tokens a warp takes an output and all the CTA's tokens, so a piece of
// the router's row is fetched once for all of them.  Then warp k chooses for token k.
template <typename T, int TOK>
__global__ void __launch_bounds__(256)
moe_route_choice_kernel(const T* __restrict__ h, const float* __restrict__ wr, const float* __restrict__ correction,
                        const int* __restrict__ token_pos, int* __restrict__ ids, float* __restrict__ weights,
                        float* __restrict__ pass_weight, int n_tokens, int width, int outputs, int experts, int top,
                        int groups, int keep) {
    extern __shared__ float z_all[];
    const int per = 2 * outputs + groups;
    pdl_wait();
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int n0 = blockIdx.x * TOK;
    const bool by_four = (width & 3) == 0;
    if (TOK == 1) {
        const T* x = h + (size_t)n0 * width;
        for (int e0 = warp; e0 < outputs; e0 += 32) {
            float acc[4] = {0.f, 0.f, 0.f, 0.f};
            const float* w[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) w[k] = wr + (size_t)min(e0 + 8 * k, outputs - 1) * width;
            if (by_four) {
#pragma unroll 2
                for (int i = lane * 4; i < width; i += 128) {
                    const float4 xv = load4(x + i);
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const float4 wv = load4(w[k] + i);
                        acc[k] = fmaf(wv.x, xv.x, acc[k]);
                        acc[k] = fmaf(wv.y, xv.y, acc[k]);
                        acc[k] = fmaf(wv.z, xv.z, acc[k]);
                        acc[k] = fmaf(wv.w, xv.w, acc[k]);
                    }
                }
            } else {
                for (int i = lane; i < width; i += 32) {
                    const float xv = to_float(x[i]);
#pragma unroll
                    for (int k = 0; k < 4; ++k) acc[k] = fmaf(w[k][i], xv, acc[k]);
                }
            }
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float sum = warp_sum(acc[k]);
                if (lane == 0 && e0 + 8 * k < outputs) z_all[e0 + 8 * k] = sum;
            }
        }
    } else {
        const T* x[TOK];
#pragma unroll
        for (int k = 0; k < TOK; ++k) x[k] = h + (size_t)min(n0 + k, n_tokens - 1) * width;
        for (int e = warp; e < outputs; e += 8) {
            const float* w = wr + (size_t)e * width;
            float acc[TOK];
#pragma unroll
            for (int k = 0; k < TOK; ++k) acc[k] = 0.f;
            if (by_four) {
#pragma unroll 2
                for (int i = lane * 4; i < width; i += 128) {
                    const float4 wv = load4(w + i);
#pragma unroll
                    for (int k = 0; k < TOK; ++k) {
                        const float4 xv = load4(x[k] + i);
                        acc[k] = fmaf(wv.x, xv.x, acc[k]);
                        acc[k] = fmaf(wv.y, xv.y, acc[k]);
                        acc[k] = fmaf(wv.z, xv.z, acc[k]);
                        acc[k] = fmaf(wv.w, xv.w, acc[k]);
                    }
                }
            } else {
                for (int i = lane; i < width; i += 32) {
                    const float wv = w[i];
#pragma unroll
                    for (int k = 0; k < TOK; ++k) acc[k] = fmaf(wv, to_float(x[k][i]), acc[k]);
                }
            }
#pragma unroll
            for (int k = 0; k < TOK; ++k) {
                const float sum = warp_sum(acc[k]);
                if (lane == 0) z_all[k * per + e] = sum;
            }
        }
    }
    __syncthreads();
    const int n = n0 + warp;
    if (warp >= TOK || n >= n_tokens) return;
    float* z = z_all + warp * per;
    float* choice = z + outputs;
    float* run_best = choice + outputs;
    int* id = ids + (size_t)n * top;
    float* wt = weights + (size_t)n * top;
    if (token_pos[n] < 0) {
        for (int s = lane; s < top; s += 32) {
            id[s] = -1;
            wt[s] = 0.f;
        }
        if (lane == 0) pass_weight[n] = 0.f;
        return;
    }
    // one softmax over all outputs
    float mx = -FLT_MAX;
    for (int e = lane; e < outputs; e += 32) mx = fmaxf(mx, z[e]);
    mx = warp_max(mx);
    float sum = 0.f;
    for (int e = lane; e < outputs; e += 32) {
        const float p = expf(z[e] - mx);
        z[e] = p;
        sum += p;
    }
    sum = warp_sum(sum);
    const float inv = 1.0f / sum;
    for (int e = lane; e < outputs; e += 32) {
        const float s = z[e] * inv;
        z[e] = s;
        choice[e] = s + (correction ? correction[e] : 0.f);
    }
    __syncwarp();
    if (groups > 1 && keep < groups) {
        const int size = outputs / groups;
        for (int g = lane; g < groups; g += 32) {
            float best = -INFINITY;
            for (int e = g * size; e < (g + 1) * size; ++e) best = fmaxf(best, choice[e]);
            run_best[g] = best;
        }
        __syncwarp();
        // the runs that are NOT among the `keep` best: a run is kept if fewer than `keep` runs beat it
        // (a run beats another with a larger score, or an equal score and a lower index)
        for (int g = lane; g < groups; g += 32) {
            const float mine = run_best[g];
            int ahead = 0;
            for (int o = 0; o < groups; ++o) ahead += (run_best[o] > mine || (run_best[o] == mine && o < g)) ? 1 : 0;
            if (ahead >= keep)
                for (int e = g * size; e < (g + 1) * size; ++e) choice[e] = -INFINITY;
        }
        __syncwarp();
    }
    float passed = 0.f;
    for (int s = 0; s < top; ++s) {
        float best = -INFINITY;
        int arg = 0x7fffffff;
        for (int e = lane; e < outputs; e += 32) {
            const float v = choice[e];
            if (v > best || (v == best && arg == 0x7fffffff && !isnan(v))) {  // (ascending e: the lower index wins a tie)
                best = v;
                arg = e;
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
            if (ob > best || (ob == best && oa < arg)) {
                best = ob;
                arg = oa;
            }
        }
        const float score = z[arg];
        if (arg >= experts) passed += score;
        __syncwarp();
        if (lane == 0) {
            id[s] = arg < experts ? arg : -1;
            wt[s] = score;
            choice[arg] = -INFINITY;  // (chosen once)
            z[arg] = 0.f;             // (a second pick of an exhausted list would weigh nothing)
        }
        __syncwarp();
    }
    if (lane == 0) pass_weight[n] = passed;
}

template <typename T>
__global__ void __launch_bounds__(256)
moe_up_kernel(const T* __restrict__ h, const T* __restrict__ w_up, const int* __restrict__ ids,
              const int* __restrict__ token_pos, T* __restrict__ act, int width, int ff, int top) {
    pdl_wait();
    pdl_launch_dependents();
    int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    long long pair = blockIdx.x;
    int f = blockIdx.y * 8 + warp;
    long long n = pair / top;
    if (f >= ff || token_pos[n] < 0) return;
    const T* w = w_up + ((size_t)ids[pair] * ff + f) * width;
    const T* x = h + (size_t)n * width;
    float acc = warp_row_dot(w, x, width, lane);
    if (lane == 0) {
        float a = fmaxf(acc, 0.f);
        act[(size_t)pair * ff + f] = from_float<T>(a * a);
    }
}

template <typename T>
__global__ void __launch_bounds__(256)
moe_up_gated_kernel(const T* __restrict__ h, const T* __restrict__ w_gu, const int* __restrict__ ids,
                    const float* __restrict__ weights, const int* __restrict__ token_pos, T* __restrict__ act,
                    int width, int ff, int top) {
    pdl_wait();
    pdl_launch_dependents();
    int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    long long pair = blockIdx.x;
    int f = blockIdx.y * 8 + warp;
    long long n = pair / top;
    if (f >= ff || token_pos[n] < 0 || ids[pair] < 0) return;
    const T* wg = w_gu + ((size_t)ids[pair] * 2 * ff + 2 * f) * width;  // (rows interleaved: gate, up)
    const T* wu = wg + width;
    const T* x = h + (size_t)n * width;
    float g = warp_row_dot(wg, x, width, lane);
    float u = warp_row_dot(wu, x, width, lane);
    if (lane == 0) {
        float w = weights ? weights[pair] : 1.0f;
        g *= w;
        u *= w;
        act[(size_t)pair * ff + f] = from_float<T>(g / (1.0f + expf(-g)) * u);
    }
}

template <typename T>
__global__ void __launch_bounds__(256)
moe_down_kernel(const T* __restrict__ act, const T* __restrict__ w_down, const int* __restrict__ ids,
                const float* __restrict__ weights, const int* __restrict__ token_pos,
                float* __restrict__ residual, int width, int ff, int top,
                const float* __restrict__ pass_weight, const T* __restrict__ h) {
    pdl_wait();
    pdl_launch_dependents();
    int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    long long n = blockIdx.x;
    int c = blockIdx.y * 8 + warp;
    if (c >= width || token_pos[n] < 0) return;
    // (what the experts that hand their input on add: their weights' sum times the input)
    float sum = pass_weight ? pass_weight[n] * to_float(h[(size_t)n * width + c]) : 0.f;
    for (int s = 0; s < top; ++s) {
        if (ids[n * top + s] < 0) continue;
        const T* w = w_down + ((size_t)ids[n * top + s] * width + c) * ff;
        const T* a = act + ((size_t)n * top + s) * ff;
        float acc = warp_row_dot(w, a, ff, lane);
        sum = weights ? fmaf(weights[n * top + s], acc, sum) : sum + acc;
    }
    if (lane == 0) residual[(size_t)n * width + c] += sum;
}

}  // namespace nnis

using namespace nnis;

NNIS_API int nnis_moe_route(const void* h, const float* wr, const float* br, const int* token_pos,
                            int* ids, float* weights, int n_tokens, int width, int experts, int top,
                            int sigmoid_scores, int dtype, cudaStream_t stream) {
    if (n_tokens <= 0 || width <= 0 || experts <= 0 || top <= 0 || top > experts || !h || !wr || !ids ||
        !weights || !token_pos)
        return NNIS_ERR_ARGUMENT;
    size_t smem = (size_t)experts * sizeof(float);
    if (smem > 48 * 1024) return NNIS_ERR_UNSUPPORTED;
    unsigned blocks = (unsigned)n_tokens;
    cudaError_t e;
    if (dtype == NNIS_DTYPE_F32)
        e = launch_dependent(moe_route_kernel<float>, blocks, 256, smem, stream, (const float*)h, wr, br, token_pos,
                             ids, weights, n_tokens, width, experts, top, sigmoid_scores);
    else if (dtype == NNIS_DTYPE_BF16)
        e = launch_dependent(moe_route_kernel<bf16>, blocks, 256, smem, stream, (const bf16*)h, wr, br, token_pos,
                             ids, weights, n_tokens, width, experts, top, sigmoid_scores);
    else
        return NNIS_ERR_UNSUPPORTED;
    return e == cudaSuccess ? NNIS_OK : (int)e;
}

// act: operand dtype [n_tokens, top, ff] (scratch); residual: float32 [n_tokens, width]
NNIS_API int nnis_moe_experts(const void* h, const void* w_up, const void* w_down, const int* ids,
                              const float* weights, const int* token_pos, void* act, float* residual,
                              int n_tokens, int width, int ff, int top, int dtype,
                              cudaStream_t stream) {
    if (n_tokens <= 0 || width <= 0 || ff <= 0 || top <= 0 || !h || !w_up || !w_down || !ids ||
        !weights || !token_pos || !act || !residual)
        return NNIS_ERR_ARGUMENT;
    if ((ff + 7) / 8 > 65535 || (width + 7) / 8 > 65535) return NNIS_ERR_UNSUPPORTED;
    dim3 up_grid((unsigned)((long long)n_tokens * top), (ff + 7) / 8);
    dim3 down_grid(n_tokens, (width + 7) / 8);
    cudaError_t e;
    if (dtype == NNIS_DTYPE_F32) {
        e = launch_dependent(moe_up_kernel<float>, up_grid, 256, 0, stream, (const float*)h, (const float*)w_up, ids,
                             token_pos, (float*)act, width, ff, top);
        if (e == cudaSuccess)
            e = launch_dependent(moe_down_kernel<float>, down_grid, 256, 0, stream, (const float*)act,
                                 (const float*)w_down, ids, weights, token_pos, residual, width, ff, top, (const float*)nullptr, (const float*)nullptr);
    } else if (dtype == NNIS_DTYPE_BF16) {
        e = launch_dependent(moe_up_kernel<bf16>, up_grid, 256, 0, stream, (const bf16*)h, (const bf16*)w_up, ids,
                             token_pos, (bf16*)act, width, ff, top);
        if (e == cudaSuccess)
            e = launch_dependent(moe_down_kernel<bf16>, down_grid, 256, 0, stream, (const bf16*)act,
                                 (const bf16*)w_down, ids, weights, token_pos, residual, width, ff, top, (const float*)nullptr, (const bf16*)nullptr);
    } else {
        return NNIS_ERR_UNSUPPORTED;
    }
    return e == cudaSuccess ? NNIS_OK : (int)e;
}

// The gated form: w_gu [experts, 2 ff, width], gate and up rows interleaved; the weights multiply
// the experts' inputs.
NNIS_API int nnis_moe_experts_gated(const void* h, const void* w_gu, const void* w_down, const int* ids,
                                    const float* weights, const int* token_pos, void* act, float* residual,
                                    int n_tokens, int width, int ff, int top, int dtype, cudaStream_t stream) {
    if (n_tokens <= 0 || width <= 0 || ff <= 0 || top <= 0 || !h || !w_gu || !w_down || !ids || !weights ||
        !token_pos || !act || !residual)
        return NNIS_ERR_ARGUMENT;
    if ((ff + 7) / 8 > 65535 || (width + 7) / 8 > 65535) return NNIS_ERR_UNSUPPORTED;
    dim3 up_grid((unsigned)((long long)n_tokens * top), (ff + 7) / 8);
    dim3 down_grid(n_tokens, (width + 7) / 8);
    cudaError_t e;
    if (dtype == NNIS_DTYPE_F32) {
        e = launch_dependent(moe_up_gated_kernel<float>, up_grid, 256, 0, stream, (const float*)h, (const float*)w_gu,
                             ids, weights, token_pos, (float*)act, width, ff, top);
        if (e == cudaSuccess)
            e = launch_dependent(moe_down_kernel<float>, down_grid, 256, 0, stream, (const float*)act,
                                 (const float*)w_down, ids, (const float*)nullptr, token_pos, residual, width, ff,
                                 top, (const float*)nullptr, (const float*)nullptr);
    } else if (dtype == NNIS_DTYPE_BF16) {
        e = launch_dependent(moe_up_gated_kernel<bf16>, up_grid, 256, 0, stream, (const bf16*)h, (const bf16*)w_gu,
                             ids, weights, token_pos, (bf16*)act, width, ff, top);
        if (e == cudaSuccess)
            e = launch_dependent(moe_down_kernel<bf16>, down_grid, 256, 0, stream, (const bf16*)act,
                                 (const bf16*)w_down, ids, (const float*)nullptr, token_pos, residual, width, ff,
                                 top, (const float*)nullptr, (const bf16*)nullptr);
    } else {
        return NNIS_ERR_UNSUPPORTED;
    }
    return e == cudaSuccess ? NNIS_OK : (int)e;
}

// The router that scores all its outputs with one softmax: see moe_route_choice above.  wr float32
// [outputs, width]; correction float32 [outputs] or null; ids int32 [n, top] (-1: an output from
// `experts` on); weights float32 [n, top]; pass_weight float32 [n].
NNIS_API int nnis_moe_route_choice(const void* h, const float* wr, const float* correction, const int* token_pos,
                                   int* ids, float* weights, float* pass_weight, int n_tokens, int width,
                                   int outputs, int experts, int top, int groups, int keep, int dtype,
                                   cudaStream_t stream) {
    if (n_tokens <= 0 || width <= 0 || outputs <= 0 || experts < 0 || experts > outputs || top <= 0 ||
        top > outputs || groups <= 0 || outputs % groups || keep <= 0 || keep > groups || !h || !wr || !ids ||
        !weights || !pass_weight || !token_pos)
        return NNIS_ERR_ARGUMENT;
    if (top > keep * (outputs / groups)) return NNIS_ERR_ARGUMENT;
    const size_t per = (2 * (size_t)outputs + groups) * sizeof(float);
    if (per > 48 * 1024) return NNIS_ERR_UNSUPPORTED;
    // many tokens: four a CTA, so a row of the router's matrix is fetched once for four of them
    const bool several = n_tokens >= 64 && 4 * per <= 48 * 1024;
    const unsigned blocks = several ? (unsigned)((n_tokens + 3) / 4) : (unsigned)n_tokens;
    const size_t smem = several ? 4 * per : per;
    cudaError_t e;
#define NNIS_ROUTE(T, TOK) \
    launch_dependent(moe_route_choice_kernel<T, TOK>, blocks, 256, smem, stream, (const T*)h, wr, correction, \
                     token_pos, ids, weights, pass_weight, n_tokens, width, outputs, experts, top, groups, keep)
    if (dtype == NNIS_DTYPE_F32)
        e = several ? NNIS_ROUTE(float, 4) : NNIS_ROUTE(float, 1);
    else if (dtype == NNIS_DTYPE_BF16)
        e = several ? NNIS_ROUTE(bf16, 4) : NNIS_ROUTE(bf16, 1);
    else
        return NNIS_ERR_UNSUPPORTED;
#undef NNIS_ROUTE
    return e == cudaSuccess ? NNIS_OK : (int)e;
}

// Gated experts whose weights multiply their OUTPUTS; a pair with a negative id has no expert;
// pass_weight (float32 [n] or null) times the token's input is added too.
NNIS_API int nnis_moe_experts_gated_out(const void* h, const void* w_gu, const void* w_down, const int* ids,
                                        const float* weights, const float* pass_weight, const int* token_pos,
                                        void* act, float* residual, int n_tokens, int width, int ff, int top,
                                        int dtype, cudaStream_t stream) {
    if (n_tokens <= 0 || width <= 0 || ff <= 0 || top <= 0 || !h || !w_gu || !w_down || !ids || !weights ||
        !token_pos || !act || !residual)
        return NNIS_ERR_ARGUMENT;
    if ((ff + 7) / 8 > 65535 || (width + 7) / 8 > 65535) return NNIS_ERR_UNSUPPORTED;
    dim3 up_grid((unsigned)((long long)n_tokens * top), (ff + 7) / 8);
    dim3 down_grid(n_tokens, (width + 7) / 8);
    cudaError_t e;
    if (dtype == NNIS_DTYPE_F32) {
        e = launch_dependent(moe_up_gated_kernel<float>, up_grid, 256, 0, stream, (const float*)h, (const float*)w_gu,
                             ids, (const float*)nullptr, token_pos, (float*)act, width, ff, top);
        if (e == cudaSuccess)
            e = launch_dependent(moe_down_kernel<float>, down_grid, 256, 0, stream, (const float*)act,
                                 (const float*)w_down, ids, weights, token_pos, residual, width, ff, top, pass_weight,
                                 (const float*)h);
    } else if (dtype == NNIS_DTYPE_BF16) {
        e = launch_dependent(moe_up_gated_kernel<bf16>, up_grid, 256, 0, stream, (const bf16*)h, (const bf16*)w_gu,
                             ids, (const float*)nullptr, token_pos, (bf16*)act, width, ff, top);
        if (e == cudaSuccess)
            e = launch_dependent(moe_down_kernel<bf16>, down_grid, 256, 0, stream, (const bf16*)act,
                                 (const bf16*)w_down, ids, weights, token_pos, residual, width, ff, top, pass_weight,
                                 (const bf16*)h);
    } else {
        return NNIS_ERR_UNSUPPORTED;
    }
    return e == cudaSuccess ? NNIS_OK : (int)e;
}
