// Prompt attention with a sink on the tensor cores, bfloat16, key and value heads of one
// size (64 or 128) over the paged cache: the prompt-step form of attention_sink.cu.
//
// A CTA of four warps owns 64 consecutive query tokens of one sequence and one query head,
// each warp 16 rows of m16n8k16 tiles.  It walks the pages (64 keys) that its rows can see:
// from the page that holds the start of the first row's chunk (or window) to the page of the
// last row.  K and V pages come into swizzled shared memory by 16-byte cp.async copies, two
// pages ahead; S = Q K^T and O += P V are matrix products; between them, in float32
// registers: score = cap * tanh(scale * s / cap) (cap 0: none), the mask (causal, the row's
// own chunk counted from position 0 of the sequence, the window), and the online softmax,
// whose running maximum starts at the head's sink and whose running sum starts at one: the
// sink's own term, which has no key and no value.  The rows leave multiplied by the gate of
// their (token, head).  The host lists the tiles (sequence, first query).
#include <float.h>

#include "mma_helpers.cuh"

namespace nnis {

constexpr int kSinkRows = 64;   // query rows per CTA
constexpr int kSinkPage = 64;
constexpr int kSinkStages = 3;

template <int D>
__global__ void __launch_bounds__(128)
attn_sink_mma_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k_cache,
                     const bf16* __restrict__ v_cache, const int* __restrict__ tiles,
                     const int* __restrict__ seq_first_row, const int* __restrict__ seq_start,
                     const int* __restrict__ seq_count, const int* __restrict__ page_table, int table_cols,
                     const float* __restrict__ sink, const float* __restrict__ gate, bf16* __restrict__ out,
                     int nq, int nkv, int window, int chunk, float scale, float cap, int gate_elems) {
    constexpr int CH = D / 8, NT = D / 8, KS = D / 16;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    bf16* q_s = reinterpret_cast<bf16*>(smem_raw);  // [64, D] swizzled
    bf16* kv_s = q_s + kSinkRows * D;               // stages x (K, V) [64, D]

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, tid = threadIdx.x;
    const int seq = tiles[2 * blockIdx.x], q0 = tiles[2 * blockIdx.x + 1];
    const int hq = blockIdx.y, hk = hq / (nq / nkv);
    const int count = seq_count[seq], start = seq_start[seq];
    const int row_base = seq_first_row[seq] + q0;
    const int rows = min(kSinkRows, count - q0);
    const int pos0 = start + q0;
    const int hi = pos0 + rows;
    int lo = window > 0 ? max(0, pos0 - window + 1) : 0;
    if (chunk > 0) lo = max(lo, (pos0 / chunk) * chunk);  // (later rows' chunks start no earlier)
    const int first_page = lo / kSinkPage, n_pages = (hi - 1) / kSinkPage - first_page + 1;
    const int* table = page_table + (size_t)seq * table_cols;
    const size_t tile_elems = (size_t)kSinkPage * D;

    auto load_page = [&](int it) {
        if (it < n_pages) {
            int page = table[first_page + it];
            const bf16* ksrc = k_cache + (size_t)(page * nkv + hk) * tile_elems;
            const bf16* vsrc = v_cache + (size_t)(page * nkv + hk) * tile_elems;
            bf16* kd = kv_s + (size_t)(it % kSinkStages) * 2 * tile_elems;
            bf16* vd = kd + tile_elems;
            for (int c = tid; c < kSinkPage * CH; c += 128) {
                int row = c / CH, part = c % CH;
                cp_async16(kd + swz<D>(row, part), ksrc + (size_t)c * 8);
                cp_async16(vd + swz<D>(row, part), vsrc + (size_t)c * 8);
            }
        }
        cp_async_commit();
    };
    for (int it = 0; it < kSinkStages - 1; ++it) load_page(it);

    for (int c = tid; c < kSinkRows * CH; c += 128) {
        int row = c / CH, part = c % CH;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (row < rows)
            v = *reinterpret_cast<const uint4*>(q + ((size_t)(row_base + row) * nq + hq) * D + part * 8);
        *reinterpret_cast<uint4*>(q_s + swz<D>(row, part)) = v;
    }
    __syncthreads();
    uint32_t qa[KS][4];
#pragma unroll
    for (int kk = 0; kk < KS; ++kk)
        ldmatrix_x4(qa[kk], q_s + swz<D>(warp * 16 + (lane & 15), kk * 2 + (lane >> 4)));

    const int r_lo = lane >> 2, c_lo = (lane & 3) * 2;
    int pos_r[2], lo_r[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        pos_r[h] = pos0 + warp * 16 + r_lo + h * 8;
        lo_r[h] = window > 0 ? pos_r[h] - window + 1 : 0;
        if (chunk > 0) lo_r[h] = max(lo_r[h], (pos_r[h] / chunk) * chunk);
    }
    float o[NT][4];
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) o[j][e] = 0.f;
    // scores are kept times log2(e); the sink is one more score, held by one lane of each row's four
    float m_run[2], l_run[2];
    m_run[0] = m_run[1] = sink ? sink[hq] * kLog2e : -INFINITY;
    l_run[0] = l_run[1] = (sink && (lane & 3) == 0) ? 1.f : 0.f;
    const float cap_in = cap > 0.f ? 2.0f * kLog2e / cap : 0.f, cap_out = cap * kLog2e;
    const float sc = scale * kLog2e;

    for (int it = 0; it < n_pages; ++it) {
        cp_async_wait<kSinkStages - 2>();
        __syncthreads();
        load_page(it + kSinkStages - 1);
        const bf16* kt = kv_s + (size_t)(it % kSinkStages) * 2 * tile_elems;
        const bf16* vt = kt + tile_elems;
        const int t0 = (first_page + it) * kSinkPage;
        // a warp whose rows all lie before this page, or whose rows' chunks all start after it,
        // has nothing to see in it
        if (t0 > pos0 + warp * 16 + 15) continue;
        if (chunk > 0 && t0 + kSinkPage <= ((pos0 + warp * 16) / chunk) * chunk) continue;

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
                ldmatrix_x4(b, kt + swz<D>(j * 8 + (lane & 7), kk * 2 + (lane >> 3)));
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
                int key = t0 + j * 8 + c_lo + (e & 1);
                bool ok = key <= pos_r[e >> 1] && key >= lo_r[e >> 1];
                float v;
                if (cap > 0.f) {  // cap * tanh(x / cap) = cap * (1 - 2 / (exp(2 x / cap) + 1))
                    float e2 = exp2f(s[j][e] * scale * cap_in);
                    v = cap_out * (1.0f - __fdividef(2.0f, e2 + 1.0f));
                } else {
                    v = s[j][e] * sc;
                }
                v = ok ? v : -INFINITY;
                s[j][e] = v;
                mx[e >> 1] = fmaxf(mx[e >> 1], v);
            }
        float alpha[2], base[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
            float mn = fmaxf(m_run[r], mx[r]);
            base[r] = mn == -INFINITY ? 0.f : mn;
            alpha[r] = exp2f(m_run[r] - base[r]);
            m_run[r] = mn;
        }
        float psum[2] = {0.f, 0.f};
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            float p0v = exp2f(s[j][0] - base[0]), p1v = exp2f(s[j][1] - base[0]);
            float p2v = exp2f(s[j][2] - base[1]), p3v = exp2f(s[j][3] - base[1]);
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
                ldmatrix_x4_trans(b, vt + swz<D>(ks * 16 + (lane & 15), jn + (lane >> 4)));
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
    float inv_a = l_run[0] > 0.f ? 1.0f / l_run[0] : 0.f;
    float inv_b = l_run[1] > 0.f ? 1.0f / l_run[1] : 0.f;
    const bool by_value = gate && gate_elems > 1;  // a gate per output value: [n, nq * D]
    if (gate && !by_value) {
        if (ra < rows) inv_a *= gate[(size_t)(row_base + ra) * nq + hq];
        if (rb < rows) inv_b *= gate[(size_t)(row_base + rb) * nq + hq];
    }
#pragma unroll
    for (int jn = 0; jn < NT; ++jn) {
        int col = hq * D + jn * 8 + c_lo;
        if (ra < rows) {
            float2 g = by_value ? *reinterpret_cast<const float2*>(gate + (size_t)(row_base + ra) * nq * D + col)
                                : make_float2(1.f, 1.f);
            *reinterpret_cast<uint32_t*>(out + (size_t)(row_base + ra) * nq * D + col) =
                pack_bf16(o[jn][0] * inv_a * g.x, o[jn][1] * inv_a * g.y);
        }
        if (rb < rows) {
            float2 g = by_value ? *reinterpret_cast<const float2*>(gate + (size_t)(row_base + rb) * nq * D + col)
                                : make_float2(1.f, 1.f);
            *reinterpret_cast<uint32_t*>(out + (size_t)(row_base + rb) * nq * D + col) =
                pack_bf16(o[jn][2] * inv_b * g.x, o[jn][3] * inv_b * g.y);
        }
    }
}

template <int D>
static int launch_sink_mma(dim3 grid, cudaStream_t stream, const bf16* q, const bf16* k, const bf16* v,
                           const int* tiles, const int* first_row, const int* start, const int* count,
                           const int* table, int cols, const float* sink, const float* gate, bf16* out, int nq,
                           int nkv, int window, int chunk, float scale, float cap, int gate_elems) {
    size_t smem = ((size_t)kSinkRows * D + (size_t)kSinkStages * 2 * kSinkPage * D) * sizeof(bf16);
    auto kernel = attn_sink_mma_kernel<D>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    kernel<<<grid, 128, smem, stream>>>(q, k, v, tiles, first_row, start, count, table, cols, sink, gate, out, nq,
                                        nkv, window, chunk, scale, cap, gate_elems);
    NNIS_RETURN_LAUNCH();
}

}  // namespace nnis

// `tiles`: int32 [n_tiles, 2] = (sequence of the batch, first query of the tile within this
// step's tokens of that sequence), 64 queries a tile.  q [n, nq * d], out [n, nq * d], caches
// [pages, nkv, 64, d]; gate float32 [n, nq] or, with gate_elems = d, [n, nq * d].  Takes d = 64 and 128 with 64-key pages; else NNIS_ERR_UNSUPPORTED.
NNIS_API int nnis_attention_sink_mma(const void* q, const void* k_cache, const void* v_cache, const int* tiles,
                                     int n_tiles, const int* seq_first_row, const int* seq_start,
                                     const int* seq_count, const int* page_table, int table_cols,
                                     const float* sink, const float* gate, void* out, int nq, int nkv, int d,
                                     int page_size, int window, int chunk, float scale, float cap, int gate_elems,
                                     cudaStream_t stream) {
    using namespace nnis;
    if (n_tiles <= 0 || nq <= 0 || nkv <= 0 || nq % nkv || table_cols <= 0 || window < 0 || chunk < 0 ||
        cap < 0.f || !tiles)
        return NNIS_ERR_ARGUMENT;
    if ((d != 64 && d != 128) || page_size != kSinkPage) return NNIS_ERR_UNSUPPORTED;
    if (nq > 65535) return NNIS_ERR_UNSUPPORTED;
    if (((uintptr_t)q | (uintptr_t)k_cache | (uintptr_t)v_cache | (uintptr_t)out) % 16) return NNIS_ERR_ALIGNMENT;
    dim3 grid(n_tiles, nq);
    if (d == 64)
        return launch_sink_mma<64>(grid, stream, (const bf16*)q, (const bf16*)k_cache, (const bf16*)v_cache, tiles,
                                   seq_first_row, seq_start, seq_count, page_table, table_cols, sink, gate,
                                   (bf16*)out, nq, nkv, window, chunk, scale, cap, gate_elems);
    return launch_sink_mma<128>(grid, stream, (const bf16*)q, (const bf16*)k_cache, (const bf16*)v_cache, tiles,
                                seq_first_row, seq_start, seq_count, page_table, table_cols, sink, gate,
                                (bf16*)out, nq, nkv, window, chunk, scale, cap, gate_elems);
}
