// Prefill attention over the paged cache (bfloat16): causal, with the queries of a prompt
// portion starting at any position of their request, keys and values read through the block
// table without gathering.
//
// The step's query tokens are cut into tiles of 64 consecutive tokens of one row (the host
// lists them: tile -> row, first token).  One CTA handles one tile for one query head: its
// 4 warps hold 16 queries each as the rows of m16n8k16 tensor-core tiles and walk the keys
// lo..last query's position in chunks of 64, double-buffered with cp.async.  Per chunk
// S = Q K^T, causal (and window) mask by absolute positions, online softmax in float32
// (base 2), O += P V.  A tile may hold a single token (a decoded token in a mixed step).
//
// Reference: the reference gathers each request's K/V into a dense tensor per layer and
// calls a library attention (acorninfer/models/qwen3.py:320-333, 367-381); the masks here are
// the same: query at position p sees keys <= p (:138-149, :377-378).
#include "mma_helpers.cuh"

#define PRE_THREADS 128
#define PRE_BM 64
#define PRE_BN 64

struct PrefillParams {
    const bf16* q;            // [tokens, q_stride]
    int64_t q_stride;
    bf16* out;                // [tokens, nq * D]
    const bf16* k_pages;
    const bf16* v_pages;
    const int* block_table;
    const int* page_base;
    const int* row_start;     // [rows + 1] offsets of the rows in the token arrays
    const int* row_pos;       // [rows] tokens of the request in the cache before the step
    const int* tiles;         // [n_tiles, 2]: row, first token of the tile relative to the row
    int table_stride, nq, nkv, logP, window;
    float scale_log2;
};

template <int D>
__global__ void __launch_bounds__(PRE_THREADS) attention_prefill_kernel(const PrefillParams p) {
    constexpr int LDS = D + 8;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* sK = reinterpret_cast<bf16*>(smem_raw);          // [2][BN][LDS]
    bf16* sV = sK + 2 * PRE_BN * LDS;

    const int tile = blockIdx.x, head = blockIdx.y;
    const int r = p.tiles[2 * tile], q0 = p.tiles[2 * tile + 1];
    const int row_tokens = p.row_start[r + 1] - p.row_start[r];
    const int n_q = min(PRE_BM, row_tokens - q0);            // queries in this tile
    const int tok0 = p.row_start[r] + q0;                    // first token (flat index)
    const int pos0 = p.row_pos[r] + q0;                      // its absolute position
    const int kvh = head / (p.nq / p.nkv);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, tq = lane & 3;
    const int lo = p.window > 0 ? max(0, pos0 - p.window + 1) : 0;
    const int hi = pos0 + n_q;                               // keys lo .. hi-1 are read by the tile
    const int* table = p.block_table + (int64_t)r * p.table_stride - p.page_base[r];

    // this warp's queries: rows g and g+8 of its 16
    const int qi0 = warp * 16 + g, qi1 = qi0 + 8;
    uint32_t qa[D / 16][4];
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int qi = (i & 1) ? qi1 : qi0;
            const int col = ks * 16 + 2 * tq + (i >> 1) * 8;
            qa[ks][i] = qi < n_q ? *reinterpret_cast<const uint32_t*>(
                                       p.q + (int64_t)(tok0 + qi) * p.q_stride + (int64_t)head * D + col)
                                 : 0u;
        }
    float o[D / 8][4];
#pragma unroll
    for (int n = 0; n < D / 8; ++n) { o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f; }
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    const int qpos[2] = {pos0 + qi0, pos0 + qi1};
    const int warp_last_pos = pos0 + min(warp * 16 + 15, n_q - 1);     // last position this warp's queries reach
    const int warp_first_lo = p.window > 0 ? max(0, pos0 + warp * 16 - p.window + 1) : 0;
    const bool warp_active = warp * 16 < n_q;

    const int n_chunks = (hi - lo + PRE_BN - 1) / PRE_BN;
    auto load_chunk = [&](int c, int stage) {
        const int key0 = lo + c * PRE_BN;
        load_kv_pair_rows<D, LDS, PRE_THREADS>(sK + stage * PRE_BN * LDS, sV + stage * PRE_BN * LDS, p.k_pages,
                                               p.v_pages, table, key0, PRE_BN, lo, hi, p.logP, p.nkv, kvh);
        cp_async_commit();
    };

    load_chunk(0, 0);
    for (int c = 0; c < n_chunks; ++c) {
        const int stage = c & 1;
        if (c + 1 < n_chunks) {
            load_chunk(c + 1, stage ^ 1);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        const int key0 = lo + c * PRE_BN;
        // skip chunks that no query of this warp may see
        if (warp_active && key0 <= warp_last_pos && key0 + PRE_BN > warp_first_lo) {
            const bf16* kbase = sK + stage * PRE_BN * LDS;
            const bf16* vbase = sV + stage * PRE_BN * LDS;
            float s[PRE_BN / 8][4];
#pragma unroll
            for (int j = 0; j < PRE_BN / 8; ++j) { s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f; }
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks) {
#pragma unroll
                for (int j2 = 0; j2 < PRE_BN / 16; ++j2) {
                    uint32_t b[4];
                    const int mat = lane >> 3, rr = lane & 7;
                    ldmatrix_x4(b, smem_addr(kbase + (j2 * 16 + (mat >> 1) * 8 + rr) * LDS + ks * 16 + (mat & 1) * 8));
                    mma_bf16_16816(s[2 * j2], qa[ks], b[0], b[1]);
                    mma_bf16_16816(s[2 * j2 + 1], qa[ks], b[2], b[3]);
                }
            }
            float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int j = 0; j < PRE_BN / 8; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int key = key0 + j * 8 + 2 * tq + (e & 1);
                    const int qp = qpos[e >> 1];
                    const bool ok = key <= qp && key < hi && (p.window <= 0 || key > qp - p.window);
                    s[j][e] = ok ? s[j][e] * p.scale_log2 : -INFINITY;
                    mx[e >> 1] = fmaxf(mx[e >> 1], s[j][e]);
                }
            float corr[2], mref[2];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const float mn = fmaxf(m_run[h], quad_max(mx[h]));
                // a query that has seen no key yet (rows beyond n_q, or a chunk wholly masked for it)
                mref[h] = mn == -INFINITY ? 0.f : mn;
                corr[h] = exp2f(m_run[h] - mref[h]);
                m_run[h] = mn;
            }
            float psum[2] = {0.f, 0.f};
#pragma unroll
            for (int j = 0; j < PRE_BN / 8; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    s[j][e] = exp2f(s[j][e] - mref[e >> 1]);
                    psum[e >> 1] += s[j][e];
                }
            l_run[0] = l_run[0] * corr[0] + psum[0];
            l_run[1] = l_run[1] * corr[1] + psum[1];
#pragma unroll
            for (int n = 0; n < D / 8; ++n) {
                o[n][0] *= corr[0]; o[n][1] *= corr[0];
                o[n][2] *= corr[1]; o[n][3] *= corr[1];
            }
#pragma unroll
            for (int kk = 0; kk < PRE_BN / 16; ++kk) {
                const uint32_t pa[4] = {pack_bf16(s[2 * kk][0], s[2 * kk][1]), pack_bf16(s[2 * kk][2], s[2 * kk][3]),
                                        pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]),
                                        pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3])};
#pragma unroll
                for (int n2 = 0; n2 < D / 16; ++n2) {
                    uint32_t b[4];
                    const int mat = lane >> 3, rr = lane & 7;
                    ldmatrix_x4_trans(b, smem_addr(vbase + (kk * 16 + (mat & 1) * 8 + rr) * LDS + n2 * 16 + (mat >> 1) * 8));
                    mma_bf16_16816(o[2 * n2], pa, b[0], b[1]);
                    mma_bf16_16816(o[2 * n2 + 1], pa, b[2], b[3]);
                }
            }
        }
        __syncthreads();
    }
    l_run[0] = quad_sum(l_run[0]);
    l_run[1] = quad_sum(l_run[1]);
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int qi = h ? qi1 : qi0;
        if (qi >= n_q) continue;
        const float inv = 1.f / l_run[h];
        bf16* orow = p.out + ((int64_t)(tok0 + qi) * p.nq + head) * D;
#pragma unroll
        for (int n = 0; n < D / 8; ++n)
            *reinterpret_cast<uint32_t*>(orow + n * 8 + 2 * tq) = pack_bf16(o[n][2 * h] * inv, o[n][2 * h + 1] * inv);
    }
}

template <int D>
static int launch_prefill(const PrefillParams& p, int n_tiles, cudaStream_t stream) {
    constexpr int LDS = D + 8;
    const size_t smem = (size_t)2 * 2 * PRE_BN * LDS * sizeof(bf16);
    static AcornPerDevice configured;
    if (!configured.seen()) {
        cudaError_t e = cudaFuncSetAttribute(attention_prefill_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured.mark();
    }
    dim3 grid(n_tiles, p.nq);
    attention_prefill_kernel<D><<<grid, PRE_THREADS, smem, stream>>>(p);
    return acorn_launch_status();
}

extern "C" int acorn_attention_prefill_supported(int nq, int nkv, int d) {
    if (nkv <= 0 || nq % nkv != 0 || nq > 65535) return 0;
    return d % 16 == 0 && d >= 16 && d <= 128;
}

extern "C" int acorn_attention_prefill(const void* q, int64_t q_stride, void* out, const void* k_pages,
                                       const void* v_pages, const int* block_table, const int* page_base,
                                       int table_stride, const int* row_start, const int* row_pos,
                                       const int* tiles, int n_tiles, int nq, int nkv, int d, int P, float scale,
                                       int window, cudaStream_t stream) {
    if (n_tiles <= 0) return 0;
    if (!acorn_attention_prefill_supported(nq, nkv, d)) return ACORN_ERR_UNSUPPORTED;
    PrefillParams p;
    p.q = (const bf16*)q; p.q_stride = q_stride; p.out = (bf16*)out;
    p.k_pages = (const bf16*)k_pages; p.v_pages = (const bf16*)v_pages;
    p.block_table = block_table; p.page_base = page_base; p.row_start = row_start; p.row_pos = row_pos;
    p.tiles = tiles; p.table_stride = table_stride; p.nq = nq; p.nkv = nkv; p.logP = acorn_log2_exact(P);
    if (p.logP < 0) return ACORN_ERR_UNSUPPORTED;   // page sizes are powers of two
    p.window = window;
    p.scale_log2 = scale * 1.4426950408889634f;
    switch (d) {
        case 16: return launch_prefill<16>(p, n_tiles, stream);
        case 32: return launch_prefill<32>(p, n_tiles, stream);
        case 48: return launch_prefill<48>(p, n_tiles, stream);
        case 64: return launch_prefill<64>(p, n_tiles, stream);
        case 80: return launch_prefill<80>(p, n_tiles, stream);
        case 96: return launch_prefill<96>(p, n_tiles, stream);
        case 112: return launch_prefill<112>(p, n_tiles, stream);
        case 128: return launch_prefill<128>(p, n_tiles, stream);
        default: return ACORN_ERR_UNSUPPORTED;
    }
}
