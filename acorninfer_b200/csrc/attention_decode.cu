// Decode attention over the paged cache (bfloat16): split-K flash decoding, one CTA per
// (token, kv head, split), all query heads of the kv head's group share every K/V tile.
//
// For the token at position p of its request the CTA reads keys lo..p
// (lo = window ? max(0, p - window + 1) : 0) of its split, 64 keys a chunk, in a three-stage
// cp.async pipeline through the block table.  The group's query heads (rep = nq / nkv <= 16) are
// the 16 rows of an m16n8k16 tensor-core tile: S = Q K^T, online softmax in float32 (base 2),
// O += P V.  Each of the 4 warps takes 16 keys of a chunk and keeps its own running
// (max, sum, O); the warps are merged through shared memory at the end.  With one split the
// result is written directly; otherwise (O normalised, log2-sum-exp) go to scratch and a
// second kernel merges the splits.  Why mma.sync and not tcgen05: the useful M is rep (4 at
// Qwen3-8B sizes), far below a tcgen05 tile, and the kernel is bound by reading K and V once.
//
// Reference for the split/merge scheme: acorninfer/ops/paged_attention.py:33-122 (one query
// head per program there, so K/V were read rep times).
#include "mma_helpers.cuh"

#define DEC_THREADS 128
#define DEC_CHUNK 64
#ifndef DEC_STAGES
#define DEC_STAGES 3
#endif

struct DecodeParams {
    const bf16* q;            // [tokens, q_stride]: query heads first in each row
    int64_t q_stride;
    bf16* out;                // [tokens, nq * D]
    const bf16* k_pages;      // [pages, nkv, P, D]
    const bf16* v_pages;
    const int* block_table;   // [rows, table_stride]
    const int* page_base;     // [rows]
    const int* token_row;     // [tokens]
    const int* positions;     // [tokens]
    const int* token_list;    // tokens handled (nullptr: 0 .. n-1)
    float* part_o;            // [n, nq, splits, D]  (splits > 1)
    float* part_lse;          // [n, nq, splits]
    int table_stride, nq, nkv, logP, window, num_splits;
    float scale_log2;         // softmax scale * log2(e)
};

template <int D>
__global__ void __launch_bounds__(DEC_THREADS) attention_decode_kernel(const DecodeParams p) {
    constexpr int LDS = D + 8;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* sK = reinterpret_cast<bf16*>(smem_raw);          // [STAGES][CHUNK][LDS]
    bf16* sV = sK + DEC_STAGES * DEC_CHUNK * LDS;          // [STAGES][CHUNK][LDS]

    pdl_wait();
    pdl_trigger();
    const int kvh = blockIdx.x, split = blockIdx.y, ti = blockIdx.z;
    const int t = p.token_list ? p.token_list[ti] : ti;
    const int r = p.token_row[t], pos = p.positions[t];
    const int rep = p.nq / p.nkv;
    const int lo = p.window > 0 ? max(0, pos - p.window + 1) : 0;
    const int hi = pos + 1;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, tq = lane & 3;

    const int n_chunks = (hi - lo + DEC_CHUNK - 1) / DEC_CHUNK;
    const int per = (n_chunks + p.num_splits - 1) / p.num_splits;
    const int c0 = split * per, c1 = min(n_chunks, c0 + per);
    if (c0 >= c1) {      // an empty split: weight zero in the merge
        for (int h = threadIdx.x; h < rep; h += DEC_THREADS)
            p.part_lse[((int64_t)ti * p.nq + kvh * rep + h) * p.num_splits + split] = -INFINITY;
        return;
    }
    const int* table = p.block_table + (int64_t)r * p.table_stride - p.page_base[r];

    // Query fragments: rows = query heads of the group (zero beyond rep), columns = head dims.
    uint32_t qa[D / 16][4];
    {
        const bf16* qrow = p.q + (int64_t)t * p.q_stride + (int64_t)kvh * rep * D;
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int row = g + (i & 1) * 8, col = ks * 16 + 2 * tq + (i >> 1) * 8;
                qa[ks][i] = row < rep ? *reinterpret_cast<const uint32_t*>(qrow + row * D + col) : 0u;
            }
        }
    }

    float o[D / 8][4];
#pragma unroll
    for (int n = 0; n < D / 8; ++n) { o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f; }
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};

    auto load_chunk = [&](int c, int stage) {
        if (c < c1)
            load_kv_pair_rows<D, LDS, DEC_THREADS>(sK + stage * DEC_CHUNK * LDS, sV + stage * DEC_CHUNK * LDS,
                                                   p.k_pages, p.v_pages, table, lo + c * DEC_CHUNK, DEC_CHUNK, lo, hi,
                                                   p.logP, p.nkv, kvh);
        cp_async_commit();      // a group per chunk slot, empty past the end, keeps the wait count fixed
    };

#pragma unroll
    for (int s = 0; s < DEC_STAGES - 1; ++s) load_chunk(c0 + s, s);
    for (int c = c0; c < c1; ++c) {
        const int stage = (c - c0) % DEC_STAGES;
        // the chunk that frees up is the one computed in the previous iteration (all warps passed
        // the barrier at its end)
        load_chunk(c + DEC_STAGES - 1, (c - c0 + DEC_STAGES - 1) % DEC_STAGES);
        cp_async_wait<DEC_STAGES - 1>();
        __syncthreads();
        const int wkey0 = lo + c * DEC_CHUNK + warp * 16;     // first key of this warp's 16
        if (wkey0 < hi) {
            const bf16* kbase = sK + (stage * DEC_CHUNK + warp * 16) * LDS;
            const bf16* vbase = sV + (stage * DEC_CHUNK + warp * 16) * LDS;
            float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks) {
                uint32_t b[4];
                const int mat = lane >> 3, rr = lane & 7;
                ldmatrix_x4(b, smem_addr(kbase + ((mat >> 1) * 8 + rr) * LDS + ks * 16 + (mat & 1) * 8));
                mma_bf16_16816(s[0], qa[ks], b[0], b[1]);
                mma_bf16_16816(s[1], qa[ks], b[2], b[3]);
            }
            float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int j = 0; j < 2; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int key = wkey0 + j * 8 + 2 * tq + (e & 1);
                    s[j][e] = key < hi ? s[j][e] * p.scale_log2 : -INFINITY;
                    mx[e >> 1] = fmaxf(mx[e >> 1], s[j][e]);
                }
            float corr[2];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const float mn = fmaxf(m_run[h], quad_max(mx[h]));     // finite: key wkey0 is valid
                corr[h] = exp2f(m_run[h] - mn);
                m_run[h] = mn;
            }
            float psum[2] = {0.f, 0.f};
#pragma unroll
            for (int j = 0; j < 2; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    s[j][e] = exp2f(s[j][e] - m_run[e >> 1]);
                    psum[e >> 1] += s[j][e];
                }
            l_run[0] = l_run[0] * corr[0] + psum[0];
            l_run[1] = l_run[1] * corr[1] + psum[1];
            uint32_t pa[4] = {pack_bf16(s[0][0], s[0][1]), pack_bf16(s[0][2], s[0][3]),
                              pack_bf16(s[1][0], s[1][1]), pack_bf16(s[1][2], s[1][3])};
#pragma unroll
            for (int n2 = 0; n2 < D / 16; ++n2) {
                uint32_t b[4];
                const int mat = lane >> 3, rr = lane & 7;
                ldmatrix_x4_trans(b, smem_addr(vbase + ((mat & 1) * 8 + rr) * LDS + n2 * 16 + (mat >> 1) * 8));
#pragma unroll
                for (int e = 0; e < 4; ++e) { o[2 * n2][e] *= corr[e >> 1]; o[2 * n2 + 1][e] *= corr[e >> 1]; }
                mma_bf16_16816(o[2 * n2], pa, b[0], b[1]);
                mma_bf16_16816(o[2 * n2 + 1], pa, b[2], b[3]);
            }
        }
        __syncthreads();
    }

    cp_async_wait<0>();
    // Merge the four warps through shared memory (the K/V buffers are free now).
    l_run[0] = quad_sum(l_run[0]);
    l_run[1] = quad_sum(l_run[1]);
    float* sm_m = reinterpret_cast<float*>(smem_raw);        // [4][16]
    float* sm_l = sm_m + 64;                                 // [4][16]
    float* sm_o = sm_l + 64;                                 // [4][16][D]
    if (tq == 0) {
        sm_m[warp * 16 + g] = m_run[0];
        sm_m[warp * 16 + g + 8] = m_run[1];
        sm_l[warp * 16 + g] = l_run[0];
        sm_l[warp * 16 + g + 8] = l_run[1];
    }
#pragma unroll
    for (int n = 0; n < D / 8; ++n) {
        float* row0 = sm_o + (warp * 16 + g) * D + n * 8 + 2 * tq;
        float* row1 = sm_o + (warp * 16 + g + 8) * D + n * 8 + 2 * tq;
        row0[0] = o[n][0]; row0[1] = o[n][1];
        row1[0] = o[n][2]; row1[1] = o[n][3];
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < rep * D; idx += DEC_THREADS) {
        const int h = idx / D, i = idx - h * D;
        float mstar = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) mstar = fmaxf(mstar, sm_m[w * 16 + h]);
        float L = 0.f, acc = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float f = exp2f(sm_m[w * 16 + h] - mstar);       // a warp without keys: exp2(-inf) = 0
            L += sm_l[w * 16 + h] * f;
            acc += sm_o[(w * 16 + h) * D + i] * f;
        }
        const int head = kvh * rep + h;
        if (p.num_splits == 1) {
            p.out[((int64_t)t * p.nq + head) * D + i] = __float2bfloat16_rn(acc / L);
        } else {
            const int64_t slot = ((int64_t)ti * p.nq + head) * p.num_splits + split;
            p.part_o[slot * D + i] = acc / L;
            if (i == 0) p.part_lse[slot] = mstar + log2f(L);
        }
    }
}

// Merges the splits of one (token, head): out = sum_s w_s o_s / sum_s w_s, w_s = 2^(lse_s - max lse).
// The first warp turns the (at most 32) log-sum-exps into weights; then each thread sums its
// head dimensions over the splits.
#define DEC_MAX_SPLITS 32

__global__ void attention_decode_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_lse,
                                              bf16* __restrict__ out, const int* __restrict__ token_list, int nq,
                                              int D, int num_splits) {
    __shared__ float wgt[DEC_MAX_SPLITS];
    pdl_wait();
    pdl_trigger();
    const int ti = blockIdx.x, head = blockIdx.y;
    const int t = token_list ? token_list[ti] : ti;
    const int64_t slot0 = ((int64_t)ti * nq + head) * num_splits;
    if (threadIdx.x < 32) {
        const float lse = threadIdx.x < num_splits ? part_lse[slot0 + threadIdx.x] : -INFINITY;
        const float mx = warp_max(lse);
        const float w = exp2f(lse - mx);                    // an empty split: exp2(-inf) = 0
        const float wsum = warp_sum(w);
        if (threadIdx.x < num_splits) wgt[threadIdx.x] = w / wsum;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < D; i += blockDim.x) {
        float acc = 0.f;
#pragma unroll 4
        for (int s = 0; s < num_splits; ++s) {
            const float w = wgt[s];
            const float v = part_o[(slot0 + s) * D + i];
            acc += w > 0.f ? w * v : 0.f;                   // an empty split left its slot unwritten
        }
        out[((int64_t)t * nq + head) * D + i] = __float2bfloat16_rn(acc);
    }
}

template <int D>
static int launch_decode(const DecodeParams& p, int n, cudaStream_t stream) {
    constexpr int LDS = D + 8;
    const size_t kv_bytes = (size_t)2 * DEC_STAGES * DEC_CHUNK * LDS * sizeof(bf16);
    const size_t merge_bytes = (size_t)(128 + 64 * D) * sizeof(float);
    const size_t smem = kv_bytes > merge_bytes ? kv_bytes : merge_bytes;
    static AcornPerDevice configured;
    if (!configured.seen()) {
        cudaError_t e = cudaFuncSetAttribute(attention_decode_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured.mark();
    }
    dim3 grid(p.nkv, p.num_splits, n);
    return acorn_launch(attention_decode_kernel<D>, grid, dim3(DEC_THREADS), smem, stream, p);
}

// The merge pass alone, for main passes that live in other files.
extern "C" int acorn_attention_decode_merge(const float* part_o, const float* part_lse, void* out,
                                            const int* token_list, int n, int nq, int d, int num_splits,
                                            cudaStream_t stream) {
    if (n <= 0 || num_splits <= 1) return 0;
    if (num_splits > DEC_MAX_SPLITS || n > 65535 || nq > 65535) return ACORN_ERR_UNSUPPORTED;
    return acorn_launch(attention_decode_merge_kernel, dim3(n, nq), dim3(d >= 128 ? 128 : 64), 0, stream, part_o,
                        part_lse, (bf16*)out, token_list, nq, d, num_splits);
}

// Sizes this kernel takes: head_dim a multiple of 16 up to 128, or 256; nq / nkv <= 16.
extern "C" int acorn_attention_decode_supported(int nq, int nkv, int d) {
    if (nkv <= 0 || nq % nkv != 0 || nq / nkv > 16) return 0;
    return (d % 16 == 0 && d >= 16 && d <= 128) || d == 256;
}

extern "C" int acorn_attention_decode(const void* q, int64_t q_stride, void* out, const void* k_pages,
                                      const void* v_pages, const int* block_table, const int* page_base,
                                      int table_stride, const int* token_row, const int* positions,
                                      const int* token_list, int n, int nq, int nkv, int d, int P, float scale,
                                      int window, int num_splits, float* part_o, float* part_lse,
                                      cudaStream_t stream) {
    if (n <= 0) return 0;
    if (!acorn_attention_decode_supported(nq, nkv, d) || num_splits < 1 || num_splits > DEC_MAX_SPLITS || n > 65535)
        return ACORN_ERR_UNSUPPORTED;
    if (num_splits > 1 && (part_o == nullptr || part_lse == nullptr)) return ACORN_ERR_UNSUPPORTED;
    DecodeParams p;
    p.q = (const bf16*)q; p.q_stride = q_stride; p.out = (bf16*)out;
    p.k_pages = (const bf16*)k_pages; p.v_pages = (const bf16*)v_pages;
    p.block_table = block_table; p.page_base = page_base; p.token_row = token_row; p.positions = positions;
    p.token_list = token_list; p.part_o = part_o; p.part_lse = part_lse;
    p.table_stride = table_stride; p.nq = nq; p.nkv = nkv; p.logP = acorn_log2_exact(P);
    if (p.logP < 0) return ACORN_ERR_UNSUPPORTED;   // page sizes are powers of two
    p.window = window; p.num_splits = num_splits;
    p.scale_log2 = scale * 1.4426950408889634f;
    int rc;
    switch (d) {
        case 16: rc = launch_decode<16>(p, n, stream); break;
        case 32: rc = launch_decode<32>(p, n, stream); break;
        case 48: rc = launch_decode<48>(p, n, stream); break;
        case 64: rc = launch_decode<64>(p, n, stream); break;
        case 80: rc = launch_decode<80>(p, n, stream); break;
        case 96: rc = launch_decode<96>(p, n, stream); break;
        case 112: rc = launch_decode<112>(p, n, stream); break;
        case 128: rc = launch_decode<128>(p, n, stream); break;
        case 256: rc = launch_decode<256>(p, n, stream); break;
        default: return ACORN_ERR_UNSUPPORTED;
    }
    if (rc != 0 || num_splits == 1) return rc;
    dim3 grid(n, nq);
    return acorn_launch(attention_decode_merge_kernel, grid, dim3(d >= 128 ? 128 : 64), 0, stream,
                        (const float*)part_o, (const float*)part_lse, (bf16*)out, token_list, nq, d, num_splits);
}
