// Mixture of experts for many tokens (prompts), bfloat16 on the tensor cores: the
// (token, chosen expert) pairs are sorted by expert, each expert's run padded to whole
// tiles of 64 rows, and the two projections run as grouped products over those tiles.
//
//   moe_sort      one CTA: counts per expert, runs padded to 64 rows, the place of every
//                 pair in the sorted order (`place`), the pair of every place (`perm`, -1
//                 for padding) and the expert of every tile (`tile_expert`, -1 past the end)
//   grouped_mma   C[tile rows, N] = A[rows] . W[expert]^T: 64 x 64 tiles, K in slices of 64
//                 through a three-stage cp.async ring into swizzled shared memory,
//                 mma.sync m16n8k16, float32 accumulation.  The first product gathers its
//                 rows from the tokens' inputs by `perm` and stores relu^2 in bfloat16; the
//                 second reads the sorted activations and stores float32.
//   moe_combine   residual[n] += sum_s weight[n, s] * y[place[n, s]], in the router's order
//
// Gated experts whose scores multiply their inputs (nnis_moe_grouped_gated): the gate's and the
// up-projection's rows are interleaved in the stacked weights (row 2f the gate's, 2f + 1 the
// up's), so a thread of the first product holds both sums of an output feature; it multiplies
// them by the pair's score and stores silu(g) * u; the combine step then adds without weights.
//
// Where an expert gets many rows (nnis_moe_grouped_tc) the runs are padded to 128 rows
// instead, moe_gather puts the tokens' inputs into the sorted order, and both products run
// on the tcgen05 kernel of the dense projections with one weight matrix per tile of rows
// (gemm_tcgen05.cu: nnis_gemm_tc_grouped), relu^2 in the first one's epilogue.
//
// A row's result depends on nothing but the row, so the order inside an expert's run
// (which the sort's atomics decide) changes no bit of the output.
#include "mma_helpers.cuh"

namespace nnis {

constexpr int kGroupRows = 64;

__global__ void __launch_bounds__(1024)
moe_sort_kernel(const int* __restrict__ ids, int n_pairs, int experts, int max_tiles, int tile_rows,
                int* __restrict__ perm, int* __restrict__ place, int* __restrict__ tile_expert) {
    extern __shared__ int sort_smem[];
    int* count = sort_smem;             // [experts]
    int* first = count + experts;       // [experts + 1]: first row of each padded run
    int* cursor = first + experts + 1;  // [experts]
    const int tid = threadIdx.x;
    for (int e = tid; e < experts; e += 1024) count[e] = cursor[e] = 0;
    for (int p = tid; p < max_tiles * tile_rows; p += 1024) perm[p] = -1;
    __syncthreads();
    for (int p = tid; p < n_pairs; p += 1024)
        if (ids[p] >= 0) atomicAdd(&count[ids[p]], 1);  // (a negative id: a pair without an expert)
    __syncthreads();
    if (tid == 0) {
        int at = 0;
        for (int e = 0; e < experts; ++e) {
            first[e] = at;
            at += (count[e] + tile_rows - 1) / tile_rows * tile_rows;
        }
        first[experts] = at;
    }
    __syncthreads();
    for (int t = tid; t < max_tiles; t += 1024) {
        int row = t * tile_rows, found = -1;
        if (row < first[experts]) {
            int lo = 0, hi = experts - 1;  // the last expert whose run starts at or before the row
            while (lo < hi) {
                int mid = (lo + hi + 1) >> 1;
                if (first[mid] <= row) lo = mid;
                else hi = mid - 1;
            }
            found = lo;
        }
        tile_expert[t] = found;
    }
    for (int p = tid; p < n_pairs; p += 1024) {
        int e = ids[p];
        if (e < 0) {
            place[p] = -1;
            continue;
        }
        int at = first[e] + atomicAdd(&cursor[e], 1);
        perm[at] = p;
        place[p] = at;
    }
}

// MODE 0: rows gathered from x by perm (pair / top), epilogue relu^2 -> bfloat16
// MODE 1: rows of a in sorted order, epilogue float32
// MODE 2: one matrix per head (blockIdx.z) on packed rows: rows 0 .. M - 1 of a, the head's
//         slice a_bs apart in a and c_bs apart in out (row stride ldc), bfloat16 out
template <int MODE>
__global__ void __launch_bounds__(128)
grouped_mma_kernel(const bf16* __restrict__ a, int lda, const int* __restrict__ perm, int top,
                   const bf16* __restrict__ w, const int* __restrict__ tile_expert,
                   void* __restrict__ out, int N, int K, int M, long long a_bs, int ldc,
                   long long c_bs, const float* __restrict__ pair_weight = nullptr) {
    constexpr int BK = 64, STAGES = 3, CH = BK / 8;
    const int expert = MODE == 2 ? (int)blockIdx.z : tile_expert[blockIdx.x];
    if (expert < 0) return;
    if (MODE == 2) a += (size_t)expert * a_bs;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    bf16* a_s = reinterpret_cast<bf16*>(smem_raw);          // stages x [64, 64]
    bf16* w_s = a_s + STAGES * kGroupRows * BK;             // stages x [64, 64]
    __shared__ int src_row[kGroupRows];
    __shared__ float row_weight[kGroupRows];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int row0 = blockIdx.x * kGroupRows, n0 = blockIdx.y * 64;
    if (tid < kGroupRows) {
        if (MODE == 2) {
            src_row[tid] = row0 + tid < M ? row0 + tid : -1;
        } else {
            int p = perm[row0 + tid];
            src_row[tid] = (MODE == 0 || MODE == 3) ? (p < 0 ? -1 : p / top) : (p < 0 ? -1 : row0 + tid);
            if (MODE == 3) row_weight[tid] = p < 0 ? 0.f : (pair_weight ? pair_weight[p] : 1.0f);
        }
    }
    __syncthreads();
    const bf16* wE = w + (size_t)expert * N * K;
    const int k_tiles = (K + BK - 1) / BK;
    auto load = [&](int kt) {
        if (kt < k_tiles) {
            bf16* ad = a_s + (size_t)(kt % STAGES) * kGroupRows * BK;
            bf16* wd = w_s + (size_t)(kt % STAGES) * kGroupRows * BK;
            const int k0 = kt * BK;
            for (int c = tid; c < kGroupRows * CH; c += 128) {
                int row = c / CH, chunk = c % CH, k = k0 + chunk * 8;
                int src = src_row[row];
                if (src >= 0 && k < K) cp_async16(ad + swz<BK>(row, chunk), a + (size_t)src * lda + k);
                else *reinterpret_cast<uint4*>(ad + swz<BK>(row, chunk)) = make_uint4(0, 0, 0, 0);
                if (n0 + row < N && k < K) cp_async16(wd + swz<BK>(row, chunk), wE + (size_t)(n0 + row) * K + k);
                else *reinterpret_cast<uint4*>(wd + swz<BK>(row, chunk)) = make_uint4(0, 0, 0, 0);
            }
        }
        cp_async_commit();
    };
    for (int kt = 0; kt < STAGES - 1; ++kt) load(kt);
    float acc[8][4];
#pragma unroll
    for (int j = 0; j < 8; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[j][e] = 0.f;
    for (int kt = 0; kt < k_tiles; ++kt) {
        cp_async_wait<STAGES - 2>();
        __syncthreads();
        load(kt + STAGES - 1);
        const bf16* at = a_s + (size_t)(kt % STAGES) * kGroupRows * BK;
        const bf16* wt = w_s + (size_t)(kt % STAGES) * kGroupRows * BK;
#pragma unroll
        for (int kk = 0; kk < BK / 16; kk += 2) {
            uint32_t a0[4], a1[4];
            ldmatrix_x4(a0, at + swz<BK>(warp * 16 + (lane & 15), kk * 2 + (lane >> 4)));
            ldmatrix_x4(a1, at + swz<BK>(warp * 16 + (lane & 15), kk * 2 + 2 + (lane >> 4)));
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                uint32_t b[4];
                ldmatrix_x4(b, wt + swz<BK>(j * 8 + (lane & 7), kk * 2 + (lane >> 3)));
                mma_bf16(acc[j], a0, b[0], b[1]);
                mma_bf16(acc[j], a1, b[2], b[3]);
            }
        }
    }
    cp_async_wait<0>();
    const int r_lo = lane >> 2, c_lo = (lane & 3) * 2;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        int r = warp * 16 + r_lo + h * 8;
        if (src_row[r] < 0) continue;
        size_t base = MODE == 2 ? (size_t)(row0 + r) * ldc + (size_t)expert * c_bs : (size_t)(row0 + r) * N;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            int col = n0 + j * 8 + c_lo;
            float v0 = acc[j][h * 2], v1 = acc[j][h * 2 + 1];
            if (MODE == 2) {
                bf16* o = reinterpret_cast<bf16*>(out);
                if (col < N) o[base + col] = __float2bfloat16_rn(v0);
                if (col + 1 < N) o[base + col + 1] = __float2bfloat16_rn(v1);
            } else if (MODE == 3) {  // (v0, v1) = (gate, up) of feature col / 2; the score on both
                const float g = v0 * row_weight[r], u = v1 * row_weight[r];
                bf16* o = reinterpret_cast<bf16*>(out);
                if (col + 1 < N) o[(size_t)(row0 + r) * (N >> 1) + (col >> 1)] =
                    __float2bfloat16_rn(g / (1.0f + __expf(-g)) * u);
            } else if (MODE == 0) {
                v0 = fmaxf(v0, 0.f);
                v1 = fmaxf(v1, 0.f);
                bf16* o = reinterpret_cast<bf16*>(out);
                if (col < N) o[base + col] = __float2bfloat16_rn(v0 * v0);
                if (col + 1 < N) o[base + col + 1] = __float2bfloat16_rn(v1 * v1);
            } else {
                float* o = reinterpret_cast<float*>(out);
                if (col < N) o[base + col] = v0;
                if (col + 1 < N) o[base + col + 1] = v1;
            }
        }
    }
}

// x_sorted[place] = x[perm[place] / top] (zeros where perm is negative): the rows of the
// first grouped product in the sorted order, for the kernel that takes its rows by TMA
__global__ void __launch_bounds__(256)
moe_gather_kernel(const bf16* __restrict__ x, const int* __restrict__ perm, int top,
                  bf16* __restrict__ x_sorted, int width) {
    pdl_wait();
    pdl_launch_dependents();
    const long long at = blockIdx.x;
    const int p = perm[at];
    const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)(p < 0 ? 0 : p / top) * width);
    uint4* dst = reinterpret_cast<uint4*>(x_sorted + (size_t)at * width);
    for (int c = threadIdx.x; c < width / 8; c += 256) dst[c] = p < 0 ? make_uint4(0, 0, 0, 0) : src[c];
}

// act[row, f] = silu(s g) * (s u) with (g, u) = up[row, 2f], up[row, 2f + 1] (float32 sums of the
// interleaved gate and up rows) and s the score of the pair that sits at the sorted row
__global__ void __launch_bounds__(256)
moe_gated_act_kernel(const float* __restrict__ up, const int* __restrict__ perm, const float* __restrict__ weights,
                     bf16* __restrict__ act, int ff) {
    pdl_wait();
    pdl_launch_dependents();
    const long long row = blockIdx.x;
    const int p = perm[row];
    const float s = p < 0 ? 0.f : (weights ? weights[p] : 1.0f);
    const float2* in = reinterpret_cast<const float2*>(up + (size_t)row * 2 * ff);
    for (int f = threadIdx.x; f < ff; f += 256) {
        float2 gu = in[f];
        float g = gu.x * s, u = gu.y * s;
        act[(size_t)row * ff + f] = __float2bfloat16_rn(p < 0 ? 0.f : g / (1.0f + __expf(-g)) * u);
    }
}

__global__ void __launch_bounds__(256)
moe_combine_kernel(const float* __restrict__ y, const int* __restrict__ place,
                   const float* __restrict__ weights, float* __restrict__ residual, int width, int top,
                   const float* __restrict__ pass_weight, const bf16* __restrict__ x) {
    const long long n = blockIdx.x;
    for (int c = threadIdx.x; c < width; c += 256) {
        // (pairs without an expert hand the token's input on: their weights' sum times the input)
        float sum = pass_weight ? pass_weight[n] * to_float(x[(size_t)n * width + c]) : 0.f;
        for (int s = 0; s < top; ++s) {
            if (place[n * top + s] < 0) continue;
            float v = y[(size_t)place[n * top + s] * width + c];
            sum = weights ? fmaf(weights[n * top + s], v, sum) : sum + v;
        }
        residual[(size_t)n * width + c] += sum;
    }
}

}  // namespace nnis

using namespace nnis;

static const size_t kGroupedSmem = (size_t)2 * 3 * kGroupRows * 64 * sizeof(bf16);

static int configure_grouped() {
    static bool configured = false;
    if (configured) return NNIS_OK;
    cudaError_t e = cudaFuncSetAttribute(grouped_mma_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)kGroupedSmem);
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(grouped_mma_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)kGroupedSmem);
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(grouped_mma_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)kGroupedSmem);
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(grouped_mma_kernel<3>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)kGroupedSmem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
    return NNIS_OK;
}

// One matrix per head on packed bfloat16 rows, on the tensor cores (what nnis_batched_linear
// computes on the CUDA cores): out[m, b * c_bs : + N] = a[m, b * a_bs : + K] . w[b]^T.  Takes
// K, lda, a_bs in multiples of 8 and 16-byte aligned a and w; else NNIS_ERR_UNSUPPORTED.
NNIS_API int nnis_batched_linear_mma(const void* a, long long lda, long long a_bs, const void* w, void* out,
                                     long long ldc, long long c_bs, int batch, int M, int N, int K,
                                     cudaStream_t stream) {
    if (!a || !w || !out || batch <= 0 || M <= 0 || N <= 0 || K <= 0) return NNIS_ERR_ARGUMENT;
    if (K % 8 || lda % 8 || a_bs % 8 || ((uintptr_t)a | (uintptr_t)w) % 16 || batch > 65535 ||
        lda > 0x7fffffff || ldc > 0x7fffffff)
        return NNIS_ERR_UNSUPPORTED;
    int code = configure_grouped();
    if (code != NNIS_OK) return code;
    dim3 grid((M + kGroupRows - 1) / kGroupRows, (N + 63) / 64, batch);
    if (grid.y > 65535u) return NNIS_ERR_UNSUPPORTED;
    grouped_mma_kernel<2><<<grid, 128, kGroupedSmem, stream>>>((const bf16*)a, (int)lda, nullptr, 1,
                                                               (const bf16*)w, nullptr, out, N, K, M, a_bs,
                                                               (int)ldc, c_bs);
    NNIS_RETURN_LAUNCH();
}

// tiles of 64 sorted rows that `n_pairs` pairs over `experts` experts may take
NNIS_API int nnis_moe_grouped_tiles(long long n_pairs, int experts) {
    return (int)((n_pairs + kGroupRows - 1) / kGroupRows) + experts;
}

NNIS_API int nnis_moe_grouped_takes(int width, int ff, int experts) {
    return width % 8 == 0 && ff % 8 == 0 && experts > 0 && (size_t)(3 * experts + 1) * sizeof(int) <= 40 * 1024;
}

// x: bfloat16 [n_tokens, width]; ids, weights [n_tokens, top] from the router (every row a
// token: no padding rows); scratch: perm int32 [tiles * 64], place int32 [n_tokens * top],
// tile_expert int32 [tiles], act bfloat16 [tiles * 64, ff], y float32 [tiles * 64, width]
// with tiles = nnis_moe_grouped_tiles(n_tokens * top, experts).
NNIS_API int nnis_moe_grouped(const void* x, const void* w_up, const void* w_down, const int* ids,
                              const float* weights, int* perm, int* place, int* tile_expert, void* act,
                              float* y, float* residual, int n_tokens, int width, int ff, int experts,
                              int top, cudaStream_t stream) {
    if (n_tokens <= 0 || top <= 0 || !x || !w_up || !w_down || !ids || !weights || !perm || !place ||
        !tile_expert || !act || !y || !residual)
        return NNIS_ERR_ARGUMENT;
    if (!nnis_moe_grouped_takes(width, ff, experts)) return NNIS_ERR_UNSUPPORTED;
    if (((uintptr_t)x | (uintptr_t)w_up | (uintptr_t)w_down | (uintptr_t)act) % 16) return NNIS_ERR_ALIGNMENT;
    const long long pairs = (long long)n_tokens * top;
    const int tiles = nnis_moe_grouped_tiles(pairs, experts);
    moe_sort_kernel<<<1, 1024, (3 * experts + 1) * sizeof(int), stream>>>(ids, (int)pairs, experts, tiles,
                                                                         kGroupRows, perm, place, tile_expert);
    const size_t smem = kGroupedSmem;
    int code = configure_grouped();
    if (code != NNIS_OK) return code;
    grouped_mma_kernel<0><<<dim3(tiles, (ff + 63) / 64), 128, smem, stream>>>(
        (const bf16*)x, width, perm, top, (const bf16*)w_up, tile_expert, act, ff, width, 0, 0, 0, 0);
    grouped_mma_kernel<1><<<dim3(tiles, (width + 63) / 64), 128, smem, stream>>>(
        (const bf16*)act, ff, perm, top, (const bf16*)w_down, tile_expert, y, width, ff, 0, 0, 0, 0);
    moe_combine_kernel<<<n_tokens, 256, 0, stream>>>(y, place, weights, residual, width, top,
                                                     (const float*)nullptr, (const bf16*)nullptr);
    NNIS_RETURN_LAUNCH();
}

// Gated experts with the scores on their inputs: w_gu [experts, 2 ff, width] with the gate's and
// the up-projection's rows interleaved; the rest as nnis_moe_grouped (act [tiles * 64, ff]).  With
// `weight_on_output` the scores weigh the experts' outputs instead (in the combine step), a pair with a
// negative id has no expert and takes no row, and pass_weight (float32 [n_tokens] or null) times the
// token's input is added.
NNIS_API int nnis_moe_grouped_gated(const void* x, const void* w_gu, const void* w_down, const int* ids,
                                    const float* weights, int* perm, int* place, int* tile_expert, void* act,
                                    float* y, float* residual, int n_tokens, int width, int ff, int experts,
                                    int top, int weight_on_output, const float* pass_weight, cudaStream_t stream) {
    if (n_tokens <= 0 || top <= 0 || !x || !w_gu || !w_down || !ids || !weights || !perm || !place ||
        !tile_expert || !act || !y || !residual)
        return NNIS_ERR_ARGUMENT;
    if (!nnis_moe_grouped_takes(width, ff, experts)) return NNIS_ERR_UNSUPPORTED;
    if (((uintptr_t)x | (uintptr_t)w_gu | (uintptr_t)w_down | (uintptr_t)act) % 16) return NNIS_ERR_ALIGNMENT;
    const long long pairs = (long long)n_tokens * top;
    const int tiles = nnis_moe_grouped_tiles(pairs, experts);
    moe_sort_kernel<<<1, 1024, (3 * experts + 1) * sizeof(int), stream>>>(ids, (int)pairs, experts, tiles,
                                                                         kGroupRows, perm, place, tile_expert);
    int code = configure_grouped();
    if (code != NNIS_OK) return code;
    grouped_mma_kernel<3><<<dim3(tiles, (2 * ff + 63) / 64), 128, kGroupedSmem, stream>>>(
        (const bf16*)x, width, perm, top, (const bf16*)w_gu, tile_expert, act, 2 * ff, width, 0, 0, 0, 0,
        weight_on_output ? (const float*)nullptr : weights);
    grouped_mma_kernel<1><<<dim3(tiles, (width + 63) / 64), 128, kGroupedSmem, stream>>>(
        (const bf16*)act, ff, perm, top, (const bf16*)w_down, tile_expert, y, width, ff, 0, 0, 0, 0);
    moe_combine_kernel<<<n_tokens, 256, 0, stream>>>(y, place, weight_on_output ? weights : (const float*)nullptr,
                                                     residual, width, top, weight_on_output ? pass_weight : nullptr,
                                                     (const bf16*)x);
    NNIS_RETURN_LAUNCH();
}

// The same with both products on the tcgen05 kernel (nnis_gemm_tc_grouped): runs padded to
// 128 rows, the first product's rows gathered into x_sorted [tiles * 128, width] first, relu^2
// in that product's epilogue.  tiles = nnis_moe_grouped_tiles_tc(n_tokens * top, experts);
// scratch as nnis_moe_grouped with 128 rows a tile, plus x_sorted (bfloat16).
NNIS_API int nnis_moe_grouped_tiles_tc(long long n_pairs, int experts) {
    return (int)((n_pairs + 127) / 128) + experts;
}

extern "C" int nnis_gemm_tc_grouped(const void* A, const void* W, void* C, int M, int N, int K, int experts,
                                    const int* tile_expert, int square_relu, int sm_count, int* status, int pdl,
                                    cudaStream_t stream);

NNIS_API int nnis_moe_grouped_tc(const void* x, const void* w_up, const void* w_down, const int* ids,
                                 const float* weights, int* perm, int* place, int* tile_expert, void* x_sorted,
                                 void* act, float* y, float* residual, int n_tokens, int width, int ff,
                                 int experts, int top, int sm_count, int* status, int pdl, cudaStream_t stream) {
    if (n_tokens <= 0 || top <= 0 || !x || !w_up || !w_down || !ids || !weights || !perm || !place ||
        !tile_expert || !x_sorted || !act || !y || !residual)
        return NNIS_ERR_ARGUMENT;
    if (!nnis_moe_grouped_takes(width, ff, experts)) return NNIS_ERR_UNSUPPORTED;
    if (((uintptr_t)x | (uintptr_t)x_sorted) % 16) return NNIS_ERR_ALIGNMENT;
    const long long pairs = (long long)n_tokens * top;
    const int tiles = nnis_moe_grouped_tiles_tc(pairs, experts);
    const int rows = tiles * 128;
    moe_sort_kernel<<<1, 1024, (3 * experts + 1) * sizeof(int), stream>>>(ids, (int)pairs, experts, tiles, 128, perm,
                                                                         place, tile_expert);
    cudaError_t e = launch_dependent(moe_gather_kernel, (unsigned)rows, 256, 0, stream, (const bf16*)x,
                                     (const int*)perm, top, (bf16*)x_sorted, width);
    if (e != cudaSuccess) return (int)e;
    int code = nnis_gemm_tc_grouped(x_sorted, w_up, act, rows, ff, width, experts, tile_expert, 1, sm_count, status,
                                    pdl, stream);
    if (code != NNIS_OK) return code;
    code = nnis_gemm_tc_grouped(act, w_down, y, rows, width, ff, experts, tile_expert, 0, sm_count, status, pdl,
                                stream);
    if (code != NNIS_OK) return code;
    moe_combine_kernel<<<n_tokens, 256, 0, stream>>>(y, place, weights, residual, width, top,
                                                     (const float*)nullptr, (const bf16*)nullptr);
    NNIS_RETURN_LAUNCH();
}

// Gated experts with the scores on their inputs, both products on the tcgen05 kernel: the first
// stores the float32 sums of the interleaved gate and up rows (`up` float32 [tiles * 128, 2 ff]),
// moe_gated_act applies score and activation, the second product and the unweighted sum follow.
NNIS_API int nnis_moe_grouped_gated_tc(const void* x, const void* w_gu, const void* w_down, const int* ids,
                                       const float* weights, int* perm, int* place, int* tile_expert,
                                       void* x_sorted, float* up, void* act, float* y, float* residual,
                                       int n_tokens, int width, int ff, int experts, int top,
                                       int weight_on_output, const float* pass_weight, int sm_count,
                                       int* status, int pdl, cudaStream_t stream) {
    if (n_tokens <= 0 || top <= 0 || !x || !w_gu || !w_down || !ids || !weights || !perm || !place ||
        !tile_expert || !x_sorted || !up || !act || !y || !residual)
        return NNIS_ERR_ARGUMENT;
    if (!nnis_moe_grouped_takes(width, ff, experts)) return NNIS_ERR_UNSUPPORTED;
    if (((uintptr_t)x | (uintptr_t)x_sorted | (uintptr_t)up) % 16) return NNIS_ERR_ALIGNMENT;
    const long long pairs = (long long)n_tokens * top;
    const int tiles = nnis_moe_grouped_tiles_tc(pairs, experts);
    const int rows = tiles * 128;
    moe_sort_kernel<<<1, 1024, (3 * experts + 1) * sizeof(int), stream>>>(ids, (int)pairs, experts, tiles, 128, perm,
                                                                         place, tile_expert);
    cudaError_t e = launch_dependent(moe_gather_kernel, (unsigned)rows, 256, 0, stream, (const bf16*)x,
                                     (const int*)perm, top, (bf16*)x_sorted, width);
    if (e != cudaSuccess) return (int)e;
    int code = nnis_gemm_tc_grouped(x_sorted, w_gu, up, rows, 2 * ff, width, experts, tile_expert, 0, sm_count, status,
                                    pdl, stream);
    if (code != NNIS_OK) return code;
    e = launch_dependent(moe_gated_act_kernel, (unsigned)rows, 256, 0, stream, (const float*)up, (const int*)perm,
                         weight_on_output ? (const float*)nullptr : weights, (bf16*)act, ff);
    if (e != cudaSuccess) return (int)e;
    code = nnis_gemm_tc_grouped(act, w_down, y, rows, width, ff, experts, tile_expert, 0, sm_count, status, pdl,
                                stream);
    if (code != NNIS_OK) return code;
    moe_combine_kernel<<<n_tokens, 256, 0, stream>>>(y, place, weight_on_output ? weights : (const float*)nullptr,
                                                     residual, width, top, weight_on_output ? pass_weight : nullptr,
                                                     (const bf16*)x);
    NNIS_RETURN_LAUNCH();
}
