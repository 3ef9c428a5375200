// Prompt attention with two maps a head on the tensor cores, bfloat16, over the paged cache: the
// prompt-step form of attention_diff.cu, for maps of 32, 64 or 128 values and values of 64 or 128.
//
// A CTA of eight warps owns 64 consecutive query tokens of one sequence and one query head.  Warps
// 0-3 compute map 1 and warps 4-7 map 2, each warp 16 rows of m16n8k16 tiles; both halves read the
// same pages from shared memory: a key page is [64, 2 dk] ([k1 | k2] a row, a half reads its own dk
// columns), a value page [64, dv] serves both.  It walks the pages that its rows can see, from the
// page that holds the start of the first row's window to the page of the last row; K and V pages
// come into swizzled shared memory by 16-byte cp.async copies, two pages ahead; S = Q K^T and
// O += P V are matrix products; between them, in float32 registers, the mask (causal, the window)
// and the online softmax.  At the end map 2's normalised rows go through shared memory to the warps
// of map 1, which form o = a1 - lambda a2, divide every row by its root mean square over the dv
// values, multiply by `post` and the gates, and store.  The host lists the tiles (sequence, first
// query).
#include <float.h>

#include "mma_helpers.cuh"

namespace nnis {

constexpr int kDiffRows = 64;   // query rows per CTA
constexpr int kDiffPage = 64;
constexpr int kDiffStages = 3;

// (small heads: two CTAs an SM, which caps a thread at 128 registers)
template <int DK, int DV>
__global__ void __launch_bounds__(256, (DK <= 64 && DV <= 64) ? 2 : 1)
attn_diff_mma_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k_cache, const bf16* __restrict__ v_cache,
                     const int* __restrict__ tiles, const int* __restrict__ seq_first_row,
                     const int* __restrict__ seq_start, const int* __restrict__ seq_count,
                     const int* __restrict__ page_table, int table_cols, const float* __restrict__ gate,
                     bf16* __restrict__ out, int nq, int nkv, int window, float scale, float lambda, float post,
                     float eps) {
    constexpr int DK2 = 2 * DK;                 // a key row, a query row
    constexpr int KCH = DK2 / 8, VCH = DV / 8;  // 16-byte chunks a row
    constexpr int NT = DV / 8, KS = DK / 16;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    bf16* q_s = reinterpret_cast<bf16*>(smem_raw);  // [64, 2 dk] swizzled
    bf16* kv_s = q_s + kDiffRows * DK2;             // stages x (K [64, 2 dk], V [64, dv])
    constexpr size_t k_elems = (size_t)kDiffPage * DK2, v_elems = (size_t)kDiffPage * DV;

    const int lane = threadIdx.x & 31, tid = threadIdx.x;
    const int warp = (threadIdx.x >> 5) & 3, map = threadIdx.x >> 7;
    const int seq = tiles[2 * blockIdx.x], q0 = tiles[2 * blockIdx.x + 1];
    const int hq = blockIdx.y, hk = hq / (nq / nkv);
    const int count = seq_count[seq], start = seq_start[seq];
    const int row_base = seq_first_row[seq] + q0;
    const int rows = min(kDiffRows, count - q0);
    const int pos0 = start + q0;
    const int hi = pos0 + rows;
    const int lo = window > 0 ? max(0, pos0 - window + 1) : 0;
    const int first_page = lo / kDiffPage, n_pages = (hi - 1) / kDiffPage - first_page + 1;
    const int* table = page_table + (size_t)seq * table_cols;

    auto load_page = [&](int it) {
        if (it < n_pages) {
            const int page = table[first_page + it];
            const bf16* ksrc = k_cache + (size_t)(page * nkv + hk) * k_elems;
            const bf16* vsrc = v_cache + (size_t)(page * nkv + hk) * v_elems;
            bf16* kd = kv_s + (size_t)(it % kDiffStages) * (k_elems + v_elems);
            bf16* vd = kd + k_elems;
            for (int c = tid; c < kDiffPage * KCH; c += 256) {
                const int row = c / KCH, part = c % KCH;
                cp_async16(kd + swz<DK2>(row, part), ksrc + (size_t)c * 8);
            }
            for (int c = tid; c < kDiffPage * VCH; c += 256) {
                const int row = c / VCH, part = c % VCH;
                cp_async16(vd + swz<DV>(row, part), vsrc + (size_t)c * 8);
            }
        }
        cp_async_commit();
    };
    for (int it = 0; it < kDiffStages - 1; ++it) load_page(it);

    for (int c = tid; c < kDiffRows * KCH; c += 256) {
        const int row = c / KCH, part = c % KCH;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (row < rows)
            v = *reinterpret_cast<const uint4*>(q + ((size_t)(row_base + row) * nq + hq) * DK2 + part * 8);
        *reinterpret_cast<uint4*>(q_s + swz<DK2>(row, part)) = v;
    }
    __syncthreads();
    uint32_t qa[KS][4];
#pragma unroll
    for (int kk = 0; kk < KS; ++kk)
        ldmatrix_x4(qa[kk], q_s + swz<DK2>(warp * 16 + (lane & 15), map * (DK / 8) + kk * 2 + (lane >> 4)));

    const int r_lo = lane >> 2, c_lo = (lane & 3) * 2;
    int pos_r[2], lo_r[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        pos_r[h] = pos0 + warp * 16 + r_lo + h * 8;
        lo_r[h] = window > 0 ? pos_r[h] - window + 1 : 0;
    }
    float o[NT][4];
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) o[j][e] = 0.f;
    // scores are kept times log2(e)
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    const float sc = scale * kLog2e;

    for (int it = 0; it < n_pages; ++it) {
        cp_async_wait<kDiffStages - 2>();
        __syncthreads();
        load_page(it + kDiffStages - 1);
        const bf16* kt = kv_s + (size_t)(it % kDiffStages) * (k_elems + v_elems);
        const bf16* vt = kt + k_elems;
        const int t0 = (first_page + it) * kDiffPage;
        // a warp whose rows all lie before this page, or whose rows' windows all start after it, has
        // nothing to see in it
        if (t0 > pos0 + warp * 16 + 15) continue;
        if (window > 0 && t0 + kDiffPage <= pos0 + warp * 16 - window + 1) continue;

        float s[8][4];
#pragma unroll
        for (int j = 0; j < 8; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) s[j][e] = 0.f;
#pragma unroll
        for (int kk = 0; kk < KS; kk += 2) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                uint32_t b[4];
                ldmatrix_x4(b, kt + swz<DK2>(j * 8 + (lane & 7), map * (DK / 8) + kk * 2 + (lane >> 3)));
                mma_bf16(s[j], qa[kk], b[0], b[1]);
                mma_bf16(s[j], qa[kk + 1], b[2], b[3]);
            }
        }
        uint32_t pa[4][4];
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int j = 0; j < 8; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int key = t0 + j * 8 + c_lo + (e & 1);
                const bool ok = key <= pos_r[e >> 1] && key >= lo_r[e >> 1];
                const float v = ok ? s[j][e] * sc : -INFINITY;
                s[j][e] = v;
                mx[e >> 1] = fmaxf(mx[e >> 1], v);
            }
        float alpha[2], base[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
            const float mn = fmaxf(m_run[r], mx[r]);
            base[r] = mn == -INFINITY ? 0.f : mn;
            alpha[r] = exp2f(m_run[r] - base[r]);
            m_run[r] = mn;
        }
        float psum[2] = {0.f, 0.f};
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float p0v = exp2f(s[j][0] - base[0]), p1v = exp2f(s[j][1] - base[0]);
            const float p2v = exp2f(s[j][2] - base[1]), p3v = exp2f(s[j][3] - base[1]);
            psum[0] += p0v + p1v;
            psum[1] += p2v + p3v;
            pa[j >> 1][(j & 1) * 2] = pack_bf16(p0v, p1v);
            pa[j >> 1][(j & 1) * 2 + 1] = pack_bf16(p2v, p3v);
        }
#pragma unroll
        for (int r = 0; r < 2; ++r) l_run[r] = l_run[r] * alpha[r] + psum[r];
#pragma unroll
        for (int jn = 0; jn < NT; ++jn)
#pragma unroll
            for (int e = 0; e < 4; ++e) o[jn][e] *= alpha[e >> 1];
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
#pragma unroll
            for (int jn = 0; jn < NT; jn += 2) {
                uint32_t b[4];
                ldmatrix_x4_trans(b, vt + swz<DV>(ks * 16 + (lane & 15), jn + (lane >> 4)));
                mma_bf16(o[jn], pa[ks], b[0], b[1]);
                mma_bf16(o[jn + 1], pa[ks], b[2], b[3]);
            }
        }
    }
    cp_async_wait<0>();
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
    }
    const int ra = warp * 16 + r_lo, rb = ra + 8;
    const float inv_a = l_run[0] > 0.f ? 1.0f / l_run[0] : 0.f;
    const float inv_b = l_run[1] > 0.f ? 1.0f / l_run[1] : 0.f;
    // map 2's rows to the warps of map 1, through the pages' place: float32 [64, dv + 8] (the eight
    // values more a row spread the rows of a warp over the banks)
    constexpr int XS = DV + 8;
    float* xch = reinterpret_cast<float*>(kv_s);
    __syncthreads();  // every warp is done with the last page
    if (map == 1) {
#pragma unroll
        for (int jn = 0; jn < NT; ++jn) {
            const int col = jn * 8 + c_lo;
            *reinterpret_cast<float2*>(xch + ra * XS + col) = make_float2(o[jn][0] * inv_a, o[jn][1] * inv_a);
            *reinterpret_cast<float2*>(xch + rb * XS + col) = make_float2(o[jn][2] * inv_b, o[jn][3] * inv_b);
        }
    }
    __syncthreads();
    if (map == 1) return;
    float ss_a = 0.f, ss_b = 0.f;
#pragma unroll
    for (int jn = 0; jn < NT; ++jn) {
        const int col = jn * 8 + c_lo;
        const float2 xa = *reinterpret_cast<const float2*>(xch + ra * XS + col);
        const float2 xb = *reinterpret_cast<const float2*>(xch + rb * XS + col);
        o[jn][0] = o[jn][0] * inv_a - lambda * xa.x;
        o[jn][1] = o[jn][1] * inv_a - lambda * xa.y;
        o[jn][2] = o[jn][2] * inv_b - lambda * xb.x;
        o[jn][3] = o[jn][3] * inv_b - lambda * xb.y;
        ss_a = fmaf(o[jn][0], o[jn][0], fmaf(o[jn][1], o[jn][1], ss_a));
        ss_b = fmaf(o[jn][2], o[jn][2], fmaf(o[jn][3], o[jn][3], ss_b));
    }
    ss_a += __shfl_xor_sync(0xffffffffu, ss_a, 1);
    ss_a += __shfl_xor_sync(0xffffffffu, ss_a, 2);
    ss_b += __shfl_xor_sync(0xffffffffu, ss_b, 1);
    ss_b += __shfl_xor_sync(0xffffffffu, ss_b, 2);
    const float unit_a = post / sqrtf(ss_a * (1.0f / (float)DV) + eps);
    const float unit_b = post / sqrtf(ss_b * (1.0f / (float)DV) + eps);
#pragma unroll
    for (int jn = 0; jn < NT; ++jn) {
        const int col = hq * DV + jn * 8 + c_lo;
        if (ra < rows) {
            const size_t at = (size_t)(row_base + ra) * nq * DV + col;
            const float2 g = gate ? *reinterpret_cast<const float2*>(gate + at) : make_float2(1.f, 1.f);
            *reinterpret_cast<uint32_t*>(out + at) = pack_bf16(o[jn][0] * unit_a * g.x, o[jn][1] * unit_a * g.y);
        }
        if (rb < rows) {
            const size_t at = (size_t)(row_base + rb) * nq * DV + col;
            const float2 g = gate ? *reinterpret_cast<const float2*>(gate + at) : make_float2(1.f, 1.f);
            *reinterpret_cast<uint32_t*>(out + at) = pack_bf16(o[jn][2] * unit_b * g.x, o[jn][3] * unit_b * g.y);
        }
    }
}

template <int DK, int DV>
static int launch_diff_mma(dim3 grid, cudaStream_t stream, const bf16* q, const bf16* k, const bf16* v,
                           const int* tiles, const int* first_row, const int* start, const int* count,
                           const int* table, int cols, const float* gate, bf16* out, int nq, int nkv, int window,
                           float scale, float lambda, float post, float eps) {
    size_t smem = ((size_t)kDiffRows * 2 * DK + (size_t)kDiffStages * kDiffPage * (2 * DK + DV)) * sizeof(bf16);
    static_assert((size_t)kDiffStages * kDiffPage * (2 * DK + DV) * sizeof(bf16) >=
                      (size_t)kDiffRows * (DV + 8) * sizeof(float),
                  "the pages' place holds map 2's rows at the end");
    auto kernel = attn_diff_mma_kernel<DK, DV>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    kernel<<<grid, 256, smem, stream>>>(q, k, v, tiles, first_row, start, count, table, cols, gate, out, nq, nkv,
                                        window, scale, lambda, post, eps);
    NNIS_RETURN_LAUNCH();
}

}  // namespace nnis

// `tiles`: int32 [n_tiles, 2] = (sequence of the batch, first query of the tile within this step's
// tokens of that sequence), 64 queries a tile.  q [n, nq * 2 dk], out [n, nq * dv], caches
// [pages, nkv, 64, 2 dk] and [pages, nkv, 64, dv]; gate float32 [n, nq * dv] or null.  Takes dk of
// 32, 64, 128 and dv of 64, 128 with 64-key pages; else NNIS_ERR_UNSUPPORTED.
NNIS_API int nnis_attention_diff_mma(const void* q, const void* k_cache, const void* v_cache, const int* tiles,
                                     int n_tiles, const int* seq_first_row, const int* seq_start,
                                     const int* seq_count, const int* page_table, int table_cols, const float* gate,
                                     void* out, int nq, int nkv, int dk, int dv, int page_size, int window,
                                     float scale, float lambda, float post, float eps, cudaStream_t stream) {
    using namespace nnis;
    if (n_tiles <= 0 || nq <= 0 || nkv <= 0 || nq % nkv || table_cols <= 0 || window < 0 || !(eps > 0.f) || !tiles ||
        !q || !k_cache || !v_cache || !out)
        return NNIS_ERR_ARGUMENT;
    if ((dk != 32 && dk != 64 && dk != 128) || (dv != 64 && dv != 128) || page_size != kDiffPage)
        return NNIS_ERR_UNSUPPORTED;
    if (nq > 65535) return NNIS_ERR_UNSUPPORTED;
    if (((uintptr_t)q | (uintptr_t)k_cache | (uintptr_t)v_cache | (uintptr_t)out | (uintptr_t)gate) % 16)
        return NNIS_ERR_ALIGNMENT;
    dim3 grid(n_tiles, nq);
#define NNIS_DIFF_MMA(DK, DV) \
    if (dk == DK && dv == DV) \
        return launch_diff_mma<DK, DV>(grid, stream, (const bf16*)q, (const bf16*)k_cache, (const bf16*)v_cache, \
                                       tiles, seq_first_row, seq_start, seq_count, page_table, table_cols, gate, \
                                       (bf16*)out, nq, nkv, window, scale, lambda, post, eps)
    NNIS_DIFF_MMA(32, 64);
    NNIS_DIFF_MMA(32, 128);
    NNIS_DIFF_MMA(64, 64);
    NNIS_DIFF_MMA(64, 128);
    NNIS_DIFF_MMA(128, 64);
    NNIS_DIFF_MMA(128, 128);
#undef NNIS_DIFF_MMA
    return NNIS_ERR_UNSUPPORTED;
}
