// Decode attention over the paged cache (bfloat16, head size 128), K and V brought by TMA.
//
// The computation is that of attention_decode.cu (split-K flash decoding, one CTA per
// (token, kv head, split), the query heads of the kv group share every K/V tile, mma.sync
// m16n8k16, online softmax in float32, warps merged through shared memory, splits merged by
// attention_decode_merge_kernel).  What differs is how K and V reach shared memory: a producer
// warp issues TMA tile loads of whole (page, kv head) tiles ([page_size x 64] boxes, two halves
// of the head dims) into a ring of stages guarded by mbarriers, so the four compute warps spend
// no instructions on addresses; the tiles land in the 128-byte swizzled layout and ldmatrix
// reads them with the matching XOR.  Chunks start at multiples of 64 keys; keys outside
// [lo, hi) are masked.  Rows of a last page beyond the request's length are read as they are
// (the cache holds finite numbers) and get probability zero.
//
// Up to sixteen splits are merged inside this kernel: the CTAs of one (token, kv head) form a
// thread-block cluster, every CTA sends its partial result of each query head (normalised output
// and log-sum) into the shared memory of the CTA that finishes that head (head h by rank h mod
// splits; remote stores through distributed shared memory), the cluster meets once, and the owners
// write the merged rows.  No scratch in global memory and no merge kernel: one kernel and one
// kernel boundary less in a decode layer.  Clusters of more than eight CTAs are the non-portable
// size the B200 allows (asked for with cudaFuncAttributeNonPortableClusterSizeAllowed).  More than
// sixteen splits (very few rows at a long context), or received rows beyond DT_RECV_MAX_BYTES, go
// through part_o / part_lse and attention_decode_merge_kernel as before.
#include <cooperative_groups.h>

#include "mma_helpers.cuh"
#include "tcgen05_helpers.cuh"

namespace cg = cooperative_groups;

#define DT_D 128
#define DT_CHUNK 64
#define DT_STAGES 3
#define DT_THREADS 160                      // 4 compute warps + 1 producer warp
#define DT_HALF_BYTES (DT_CHUNK * 128)      // [64 keys][64 dims] bf16
#define DT_STAGE_BYTES (4 * DT_HALF_BYTES)  // K half 0, K half 1, V half 0, V half 1

__device__ int g_attn_dec_tma_error = 0;

struct DecodeTmaParams {
    const bf16* q;
    int64_t q_stride;
    bf16* out;
    const int* block_table;
    const int* page_base;
    const int* token_row;
    const int* positions;
    const int* token_list;
    float* part_o;
    float* part_lse;
    int table_stride, nq, nkv, logP, window, num_splits;
    float scale_log2;
    int cluster_merge;       // 1: the splits of a (token, kv head) are a cluster and merge through shared memory
};

#define DT_RECV_ROW (DT_D + 4)              // floats a received partial row takes: the output, then its log-sum
#define DT_CLUSTER_MAX 16
#define DT_RECV_MAX_BYTES (32 * 1024)

// byte offset of the 16-byte segment `seg` (0..15 over the 128 head dims) of key row `key` inside a
// K or V stage region (two swizzled halves of [64][128 bytes])
__device__ __forceinline__ uint32_t dt_swz(int key, int seg) {
    return (uint32_t)((seg >> 3) * DT_HALF_BYTES + key * 128 + (((seg & 7) ^ (key & 7)) << 4));
}

__global__ void __launch_bounds__(DT_THREADS) attention_decode_tma_kernel(const __grid_constant__ CUtensorMap map_k,
                                                                         const __grid_constant__ CUtensorMap map_v,
                                                                         const DecodeTmaParams p) {
    extern __shared__ __align__(1024) uint8_t smem[];
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + DT_STAGES * DT_STAGE_BYTES);
    const uint32_t full0 = tc_smem(bars), empty0 = tc_smem(bars + DT_STAGES);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (tc_smem(smem) & 1023u) {
        if (threadIdx.x == 0) tc_fail(&g_attn_dec_tma_error, 9, ACORN_KERNEL_ATTN_DECODE_TMA);
        return;
    }
    if (threadIdx.x == 0) {
        for (int s = 0; s < DT_STAGES; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 4); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    // every CTA of the cluster says that it runs; nobody writes into a peer's shared memory before all have
    if (p.cluster_merge) cg::this_cluster().barrier_arrive();
    // What follows up to pdl_wait() reads only the step's own arrays (token list, rows, positions,
    // block tables: written by the host before the step), not what the kernel before this one
    // produces (the queries and the newest keys and values): the chain of dependent lookups that
    // ends in the first cache rows runs while that kernel finishes.

    const int kvh = blockIdx.x, split = blockIdx.y, ti = blockIdx.z;
    const int t = p.token_list ? p.token_list[ti] : ti;
    const int r = p.token_row[t], pos = p.positions[t];
    const int rep = p.nq / p.nkv;
    const int lo = p.window > 0 ? max(0, pos - p.window + 1) : 0;
    const int hi = pos + 1;
    const int base_key = lo & ~(DT_CHUNK - 1);                      // chunks start at multiples of 64 keys
    const int n_chunks = (hi - base_key + DT_CHUNK - 1) / DT_CHUNK;
    const int per = (n_chunks + p.num_splits - 1) / p.num_splits;
    const int c0 = split * per, c1 = min(n_chunks, c0 + per);
    if (c0 >= c1 && !p.cluster_merge) {
        pdl_wait();
        pdl_trigger();
        for (int h = threadIdx.x; h < rep; h += DT_THREADS)
            p.part_lse[((int64_t)ti * p.nq + kvh * rep + h) * p.num_splits + split] = -INFINITY;
        return;
    }

    float o[DT_D / 8][4];
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    const int g = lane >> 2, tq = lane & 3;

    if (warp == 4) {
        // ---------------------------------------------------------------- producer
        // The whole warp: lane l looks up the cache rows of the l-th TMA box (one page or 64 keys)
        // of a batch of 32 boxes, a batch ahead of the loads, so that the block-table reads cost
        // one memory latency a batch; an elected lane issues the loads.
        const int* table = p.block_table + (int64_t)r * p.table_stride - p.page_base[r];
        const int P = 1 << p.logP;
        const int rows_per_op = P < DT_CHUNK ? P : DT_CHUNK;
        const int log_ops = 6 - (p.logP < 6 ? p.logP : 6);             // boxes a chunk: 64 / rows_per_op
        const int n_ops = (c1 - c0) << log_ops;
        const int first_key = p.page_base[r] << p.logP;
        auto row_of = [&](int idx) -> int {                              // box idx of this CTA's chunks
            int key = base_key + c0 * DT_CHUNK + (idx < n_ops ? idx : 0) * rows_per_op;
            if (key >= hi) key = hi - 1 - ((hi - 1) & (rows_per_op - 1));  // masked later: any rows that exist
            if (key < first_key) key = first_key;
            const int page = table[key >> p.logP];
            return ((page * p.nkv + kvh) << p.logP) + (key & (P - 1));
        };
        int rows_next = row_of(lane);
        pdl_wait();
        pdl_trigger();
        bool good = true;
        for (int b0 = 0; b0 < n_ops && good; b0 += 32) {
            const int rows_cur = rows_next;
            if (b0 + 32 < n_ops) rows_next = row_of(b0 + 32 + lane);
            const int n_here = min(32, n_ops - b0);
            for (int l = 0; l < n_here; ++l) {
                const int idx = b0 + l, i = idx >> log_ops, k = idx & ((1 << log_ops) - 1), s = i % DT_STAGES;
                if (k == 0) {                                            // first box of a chunk: its stage must be free
                    bool got = mbar_wait(empty0 + 8 * s, ((i / DT_STAGES) & 1) ^ 1);
                    if (!got && lane == 0) tc_fail(&g_attn_dec_tma_error, 1, ACORN_KERNEL_ATTN_DECODE_TMA);
                    good = __all_sync(0xffffffffu, got);
                    if (!good) break;
                    if (elect_one()) mbar_expect_tx(full0 + 8 * s, DT_STAGE_BYTES);
                }
                const int row = __shfl_sync(0xffffffffu, rows_cur, l);
                if (elect_one()) {
                    const uint32_t dst = tc_smem(smem + s * DT_STAGE_BYTES) + (uint32_t)(k * rows_per_op) * 128;
                    tma_load_2d(dst, &map_k, full0 + 8 * s, 0, row);
                    tma_load_2d(dst + DT_HALF_BYTES, &map_k, full0 + 8 * s, 64, row);
                    tma_load_2d(dst + 2 * DT_HALF_BYTES, &map_v, full0 + 8 * s, 0, row);
                    tma_load_2d(dst + 3 * DT_HALF_BYTES, &map_v, full0 + 8 * s, 64, row);
                }
            }
        }
    } else {
        // ---------------------------------------------------------------- compute warps
        pdl_wait();
        pdl_trigger();
        uint32_t qa[DT_D / 16][4];
        {
            const bf16* qrow = p.q + (int64_t)t * p.q_stride + (int64_t)kvh * rep * DT_D;
#pragma unroll
            for (int ks = 0; ks < DT_D / 16; ++ks)
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int row = g + (i & 1) * 8, col = ks * 16 + 2 * tq + (i >> 1) * 8;
                    qa[ks][i] = row < rep ? *reinterpret_cast<const uint32_t*>(qrow + row * DT_D + col) : 0u;
                }
        }
#pragma unroll
        for (int n = 0; n < DT_D / 8; ++n) { o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f; }
        bool good = true;
        for (int c = c0; c < c1; ++c) {
            const int i = c - c0, s = i % DT_STAGES;
            if (good && !mbar_wait(full0 + 8 * s, (i / DT_STAGES) & 1)) { tc_fail(&g_attn_dec_tma_error, 2, ACORN_KERNEL_ATTN_DECODE_TMA); good = false; }
            good = __all_sync(0xffffffffu, good);
            if (!good) break;
            const int wkey0 = base_key + c * DT_CHUNK + warp * 16;      // first key of this warp's 16
            if (wkey0 < hi && wkey0 + 15 >= lo) {
                const uint32_t kb = tc_smem(smem + s * DT_STAGE_BYTES);
                const uint32_t vb = kb + 2 * DT_HALF_BYTES;
                const int mat = lane >> 3, rr = lane & 7;
                float sc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
                for (int ks = 0; ks < DT_D / 16; ++ks) {
                    uint32_t b[4];
                    ldmatrix_x4(b, kb + dt_swz(warp * 16 + (mat >> 1) * 8 + rr, ks * 2 + (mat & 1)));
                    mma_bf16_16816(sc[0], qa[ks], b[0], b[1]);
                    mma_bf16_16816(sc[1], qa[ks], b[2], b[3]);
                }
                float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
                for (int j = 0; j < 2; ++j)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int key = wkey0 + j * 8 + 2 * tq + (e & 1);
                        sc[j][e] = (key < hi && key >= lo) ? sc[j][e] * p.scale_log2 : -INFINITY;
                        mx[e >> 1] = fmaxf(mx[e >> 1], sc[j][e]);
                    }
                float corr[2];
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const float mn = fmaxf(m_run[h], quad_max(mx[h]));  // finite: the group holds a valid key
                    corr[h] = exp2f(m_run[h] - mn);
                    m_run[h] = mn;
                }
                float psum[2] = {0.f, 0.f};
#pragma unroll
                for (int j = 0; j < 2; ++j)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        sc[j][e] = exp2f(sc[j][e] - m_run[e >> 1]);
                        psum[e >> 1] += sc[j][e];
                    }
                l_run[0] = l_run[0] * corr[0] + psum[0];
                l_run[1] = l_run[1] * corr[1] + psum[1];
                const uint32_t pa[4] = {pack_bf16(sc[0][0], sc[0][1]), pack_bf16(sc[0][2], sc[0][3]),
                                        pack_bf16(sc[1][0], sc[1][1]), pack_bf16(sc[1][2], sc[1][3])};
#pragma unroll
                for (int n2 = 0; n2 < DT_D / 16; ++n2) {
                    uint32_t b[4];
                    ldmatrix_x4_trans(b, vb + dt_swz(warp * 16 + (mat & 1) * 8 + rr, n2 * 2 + (mat >> 1)));
#pragma unroll
                    for (int e = 0; e < 4; ++e) { o[2 * n2][e] *= corr[e >> 1]; o[2 * n2 + 1][e] *= corr[e >> 1]; }
                    mma_bf16_16816(o[2 * n2], pa, b[0], b[1]);
                    mma_bf16_16816(o[2 * n2 + 1], pa, b[2], b[3]);
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(empty0 + 8 * s);
        }
        l_run[0] = quad_sum(l_run[0]);
        l_run[1] = quad_sum(l_run[1]);
    }
    // every stage has been consumed (the compute warps waited for each); the ring is free for the merge
    __syncthreads();
    float* sm_m = reinterpret_cast<float*>(smem);            // [4][16]
    float* sm_l = sm_m + 64;                                 // [4][16]
    float* sm_o = sm_l + 64;                                 // [4][16][128]
    if (warp < 4) {
        if (tq == 0) {
            sm_m[warp * 16 + g] = m_run[0];
            sm_m[warp * 16 + g + 8] = m_run[1];
            sm_l[warp * 16 + g] = l_run[0];
            sm_l[warp * 16 + g + 8] = l_run[1];
        }
#pragma unroll
        for (int n = 0; n < DT_D / 8; ++n) {
            float* row0 = sm_o + (warp * 16 + g) * DT_D + n * 8 + 2 * tq;
            float* row1 = sm_o + (warp * 16 + g + 8) * DT_D + n * 8 + 2 * tq;
            row0[0] = o[n][0]; row0[1] = o[n][1];
            row1[0] = o[n][2]; row1[1] = o[n][3];
        }
    }
    __syncthreads();
    // received partial rows: recv[rank of the sender][slot][DT_RECV_ROW], behind the ring and its barriers
    float* recv = reinterpret_cast<float*>(bars + 2 * DT_STAGES + 2);
    const int csize = p.cluster_merge ? p.num_splits : 1;
    const int slots = (rep + csize - 1) / csize;
    if (p.cluster_merge) cg::this_cluster().barrier_wait();
    for (int idx = threadIdx.x; idx < rep * DT_D; idx += DT_THREADS) {
        const int h = idx / DT_D, i = idx - h * DT_D;
        float mstar = -INFINITY;
        if (c0 < c1) {
#pragma unroll
            for (int w = 0; w < 4; ++w) mstar = fmaxf(mstar, sm_m[w * 16 + h]);
        }
        float L = 0.f, acc = 0.f;
        if (c0 < c1) {
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                const float f = exp2f(sm_m[w * 16 + h] - mstar);
                L += sm_l[w * 16 + h] * f;
                acc += sm_o[(w * 16 + h) * DT_D + i] * f;
            }
        }
        const int head = kvh * rep + h;
        if (p.num_splits == 1) {
            p.out[((int64_t)t * p.nq + head) * DT_D + i] = __float2bfloat16_rn(acc / L);
        } else if (p.cluster_merge) {
            // to the CTA that finishes this head; a split without keys sends a log-sum of -inf
            const uint32_t dst = cluster_map(tc_smem(recv + ((split * slots + h / csize) * DT_RECV_ROW)), h % csize);
            st_cluster_f32(dst + 4 * i, c0 < c1 ? acc / L : 0.f);
            if (i == 0) st_cluster_f32(dst + 4 * DT_D, c0 < c1 ? mstar + log2f(L) : -INFINITY);
        } else {
            const int64_t slot = ((int64_t)ti * p.nq + head) * p.num_splits + split;
            p.part_o[slot * DT_D + i] = acc / L;
            if (i == 0) p.part_lse[slot] = mstar + log2f(L);
        }
    }
    if (p.cluster_merge) {
        cg::this_cluster().sync();                       // all partial rows have arrived
        // the heads this CTA finishes: rank, rank + csize, ...; the splits in rank order
        for (int idx = threadIdx.x; idx < slots * DT_D; idx += DT_THREADS) {
            const int slot = idx / DT_D, i = idx - slot * DT_D;
            const int h = split + slot * csize;
            if (h >= rep) break;
            float mstar = -INFINITY;
            for (int q = 0; q < csize; ++q) mstar = fmaxf(mstar, recv[(q * slots + slot) * DT_RECV_ROW + DT_D]);
            float L = 0.f, acc = 0.f;
            for (int q = 0; q < csize; ++q) {
                const float lse = recv[(q * slots + slot) * DT_RECV_ROW + DT_D];
                const float f = lse == -INFINITY ? 0.f : exp2f(lse - mstar);
                L += f;
                acc += f * recv[(q * slots + slot) * DT_RECV_ROW + i];
            }
            p.out[((int64_t)t * p.nq + kvh * rep + h) * DT_D + i] = __float2bfloat16_rn(acc / L);
        }
    }
}

// Splits up to which a call with these sizes and no scratch merges inside the kernel (1: none).
extern "C" int acorn_attention_decode_tma_merges(int nq, int nkv) {
    if (nkv <= 0 || nq % nkv) return 1;
    const int rep = nq / nkv;
    int best = 1;
    for (int s = 2; s <= DT_CLUSTER_MAX; ++s)
        if ((size_t)s * ((rep + s - 1) / s) * DT_RECV_ROW * sizeof(float) <= DT_RECV_MAX_BYTES) best = s;
    return best;
}

extern "C" int acorn_attention_decode_tma_supported(int nq, int nkv, int d, int P) {
    return nkv > 0 && nq % nkv == 0 && nq / nkv <= 16 && d == DT_D && P >= 8 && (P & (P - 1)) == 0;
}

// The main pass only: the caller merges the splits (attention_decode_merge_kernel) when num_splits > 1.
extern "C" int acorn_attention_decode_tma_main(const void* q, int64_t q_stride, void* out, const void* k_pages,
                                               const void* v_pages, int64_t num_pages, const int* block_table,
                                               const int* page_base, int table_stride, const int* token_row,
                                               const int* positions, const int* token_list, int n, int nq, int nkv,
                                               int d, int P, float scale, int window, int num_splits, float* part_o,
                                               float* part_lse, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (!acorn_attention_decode_tma_supported(nq, nkv, d, P) || num_splits < 1 || num_splits > 32 || n > 65535)
        return ACORN_ERR_UNSUPPORTED;
    // two to sixteen splits without scratch: merged inside the kernel by a cluster
    const int rep = nq / nkv;
    const size_t recv_need = (size_t)num_splits * ((rep + num_splits - 1) / num_splits) * DT_RECV_ROW * sizeof(float);
    const int cluster_merge = num_splits > 1 && num_splits <= DT_CLUSTER_MAX && recv_need <= DT_RECV_MAX_BYTES &&
                              part_o == nullptr && part_lse == nullptr;
    if (num_splits > 1 && !cluster_merge && (part_o == nullptr || part_lse == nullptr)) return ACORN_ERR_UNSUPPORTED;
    DecodeTmaParams p;
    p.q = (const bf16*)q; p.q_stride = q_stride; p.out = (bf16*)out; p.block_table = block_table;
    p.page_base = page_base; p.token_row = token_row; p.positions = positions; p.token_list = token_list;
    p.part_o = part_o; p.part_lse = part_lse; p.table_stride = table_stride; p.nq = nq; p.nkv = nkv;
    p.logP = acorn_log2_exact_tc(P); p.window = window; p.num_splits = num_splits;
    p.scale_log2 = scale * 1.4426950408889634f;
    p.cluster_merge = cluster_merge;
    CUtensorMap mk, mv;
    const int box_rows = P < DT_CHUNK ? P : DT_CHUNK;
    int rc = make_map(&mk, k_pages, num_pages * nkv * P, d, d, 64, box_rows);
    if (rc) return rc;
    rc = make_map(&mv, v_pages, num_pages * nkv * P, d, d, 64, box_rows);
    if (rc) return rc;
    const size_t recv = cluster_merge ? recv_need : 0;
    const size_t smem = (size_t)DT_STAGES * DT_STAGE_BYTES + 2 * DT_STAGES * 8 + 16 + recv;
    const size_t smem_max = (size_t)DT_STAGES * DT_STAGE_BYTES + 2 * DT_STAGES * 8 + 16 + DT_RECV_MAX_BYTES;
    static AcornPerDevice configured;
    if (!configured.seen()) {
        cudaError_t e = cudaFuncSetAttribute(attention_decode_tma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)smem_max);
        if (e != cudaSuccess) return (int)e;
        e = cudaFuncSetAttribute(attention_decode_tma_kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
        if (e != cudaSuccess) return (int)e;
        configured.mark();
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(nkv, num_splits, n);
    cfg.blockDim = dim3(DT_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = cluster_merge ? num_splits : 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = acorn_pdl_enabled() ? 2 : 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, attention_decode_tma_kernel, mk, mv, p);
    return e != cudaSuccess ? (int)e : acorn_launch_status();
}

extern "C" int acorn_attention_decode_tma_error() {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_attn_dec_tma_error, sizeof(int)) != cudaSuccess) return -1;
    if (v != 0) cudaMemcpyToSymbol(g_attn_dec_tma_error, &zero, sizeof(int));
    return v;
}

ACORN_ERROR_WORD_SETTER(acorn_attention_decode_tma_set_error_word)
