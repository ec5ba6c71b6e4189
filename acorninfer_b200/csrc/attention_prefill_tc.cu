// Prefill attention on the 5th-generation tensor cores (tcgen05), head size 128, bfloat16:
// causal attention of a tile of 128 consecutive queries of one request against its keys and
// values in the paged cache, S = Q K^T and O += P V computed by tcgen05.mma with the accumulators
// in tensor memory, K/V/Q tiles brought by TMA through the block table.
//
// One CTA per (tile of 128 queries, pair of query heads that share a key/value head), one CTA to
// an SM.  The two heads ("units") read the same K/V tiles, which are loaded once, and take turns
// on the tensor cores: while the softmax warps of one unit work on a block of 128 keys, the
// tensor cores add P V of the other unit's block and compute its next scores.  With an odd
// number of query heads per key/value head the last CTA of a group has one unit only.
//   warps 0-3  softmax of unit 0, warps 4-7 of unit 1: thread r owns query row r (= TMEM lane r):
//              reads its row of S with tcgen05.ld, masks by absolute position (causal, window)
//              where a block needs it, exponentiates in float32 base 2 against a reference
//              maximum and writes P (bfloat16, two keys to a column) over the first half of S
//              with tcgen05.st.  O stays in tensor memory across blocks; it is rescaled
//              (tcgen05.ld / st) only when a row's maximum has grown by more than 2^8 since its
//              reference was set, so most blocks skip that pass.  At the end the thread reads
//              its row of O, divides by the row sum and writes the output.
//   warp 8     producer: TMA loads of Q (once) and of the K and V tiles of each block
//              ((page, kv head) tiles are contiguous [page_size x 128] in the cache) into a ring
//              of five 32 KB slots, K_0 V_0 K_1 V_1 ..., so that loads run two blocks ahead.
//   warp 9     MMA issuer (converged; one elected lane issues): per block j and unit u,
//              O_u += P_u[j] V_j with P as the A operand from tensor memory, then
//              S_u = Q_u K_{j+1}^T into the columns P_u[j] was read from (the tensor pipe runs
//              the products in the order they were issued).
// Tensor memory (512 columns): S / P of unit u at columns 128 u, O of unit u at 256 + 128 u.
// V is the MN-major B operand of the second product (head dims contiguous).
//
// Every mbarrier wait is bounded; a wait that gives up records g_attn_tc_error and the CTA
// drains without touching tensor memory it does not own.
#include "tcgen05_helpers.cuh"

#define ATC_D 128
#define ATC_BM 128
#define ATC_BN 128
#define ATC_SLOTS 5
#define ATC_THREADS 320
#define ATC_RESCALE_LOG2 8.0f     // rescale O only when the row maximum grew by more than this (base 2)

__device__ int g_attn_tc_error = 0;

struct AttnTcParams {
    bf16* out;               // [tokens, nq * 128]
    const int* block_table;
    const int* page_base;
    const int* row_start;
    const int* row_pos;
    const int* tiles;        // [n_tiles, 2]: row, first token of the tile within the row
    int table_stride, nq, nkv, logP, window;
    int n_tiles, pairs;      // pairs = ceil((nq / nkv) / 2): CTAs per (tile, kv head)
    float scale_log2;
};

// shared memory map (bytes; the tile regions are 1024-aligned)
#define ATC_Q_BYTES (2 * ATC_BM * 128)                    // one unit: two 64-element halves of [128 x 128]
#define ATC_HALF_BYTES (ATC_BN * 128)                      // one half of a K or V tile: [128 keys x 64 dims]
#define ATC_TILE_BYTES (2 * ATC_HALF_BYTES)
#define ATC_SMEM_TILES (2 * ATC_Q_BYTES + ATC_SLOTS * ATC_TILE_BYTES)
// q_full, full[SLOTS], empty[SLOTS], s_full[unit], p_full[unit], o_done[unit]
#define ATC_NUM_BARS (1 + 2 * ATC_SLOTS + 2 + 2 + 2)
#define ATC_TMEM_COLS 512

// -inf where the query at qpos may not see the key (causal, window, rows beyond the tile's queries)
__device__ __forceinline__ void atc_mask(float (&s)[64], int key0, int qpos, bool row_ok, int window) {
#pragma unroll
    for (int c = 0; c < 64; ++c) {
        const int key = key0 + c;
        const bool okk = key <= qpos && row_ok && (window <= 0 || key > qpos - window);
        s[c] = okk ? s[c] : -INFINITY;
    }
}

__device__ __forceinline__ float atc_max(const float (&s)[64]) {
    float m[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
    for (int c = 0; c < 64; c += 4) {
        m[0] = fmaxf(m[0], s[c]); m[1] = fmaxf(m[1], s[c + 1]);
        m[2] = fmaxf(m[2], s[c + 2]); m[3] = fmaxf(m[3], s[c + 3]);
    }
    return fmaxf(fmaxf(m[0], m[1]), fmaxf(m[2], m[3]));
}

// w[i] = bf16x2(2^(s[2i] * scale - ref), 2^(s[2i+1] * scale - ref)); returns the sum of the 64 values
__device__ __forceinline__ float atc_exp_pack(const float (&s)[64], float scale_log2, float neg_ref, uint32_t (&w)[32]) {
    float ps[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int c = 0; c < 64; c += 2) {
        const float a = fast_exp2(fmaf(s[c], scale_log2, neg_ref));
        const float b = fast_exp2(fmaf(s[c + 1], scale_log2, neg_ref));
        ps[(c >> 1) & 3] += a + b;
        __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
        w[c >> 1] = *reinterpret_cast<uint32_t*>(&v);
    }
    return (ps[0] + ps[1]) + (ps[2] + ps[3]);
}

__global__ void __launch_bounds__(ATC_THREADS, 1) attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q,
                                                                              const __grid_constant__ CUtensorMap map_k,
                                                                              const __grid_constant__ CUtensorMap map_v,
                                                                              const AttnTcParams p) {
    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t* sQ = smem;
    uint8_t* sKV = sQ + 2 * ATC_Q_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(sKV + ATC_SLOTS * ATC_TILE_BYTES);
    const uint32_t q_full = tc_smem(bars);
    const uint32_t full0 = q_full + 8, empty0 = full0 + 8 * ATC_SLOTS;
    const uint32_t s_full0 = empty0 + 8 * ATC_SLOTS, p_full0 = s_full0 + 16, o_done0 = p_full0 + 16;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + ATC_NUM_BARS);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // CTAs are started in the order of the tile list, which the caller sorts by falling number of keys
    // a tile reads: the long tiles first, the short ones fill the tail of the last wave.  CTAs next
    // to one another share a tile and mostly a key/value head.
    const int per_tile = p.nkv * p.pairs;
    const int tile = (int)(blockIdx.x / per_tile);
    const int kvh = (int)(blockIdx.x % per_tile) / p.pairs, pair = (int)(blockIdx.x % per_tile) % p.pairs;
    const int rep = p.nq / p.nkv;
    const int head0 = kvh * rep + 2 * pair;
    const int units = (2 * pair + 1 < rep) ? 2 : 1;
    if (tc_smem(smem) & 1023u) {            // the swizzled tiles need a 1024-byte aligned base
        if (threadIdx.x == 0) tc_fail(&g_attn_tc_error, 9, ACORN_KERNEL_ATTN_PREFILL_TC);
        return;
    }

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int s = 0; s < ATC_SLOTS; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
        for (int u = 0; u < 2; ++u) {
            mbar_init(s_full0 + 8 * u, 1); mbar_init(p_full0 + 8 * u, 4); mbar_init(o_done0 + 8 * u, 1);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 9) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     :: "r"(tc_smem(tmem_slot)), "r"((uint32_t)ATC_TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_s = tmem_base, tmem_o = tmem_base + 256;

    pdl_wait();
    pdl_trigger();
    const int r = p.tiles[2 * tile], q0 = p.tiles[2 * tile + 1];
    const int row_tokens = p.row_start[r + 1] - p.row_start[r];
    const int n_q = min(ATC_BM, row_tokens - q0);
    const int tok0 = p.row_start[r] + q0;
    const int pos0 = p.row_pos[r] + q0;
    const int hi = pos0 + n_q;                                           // keys < hi are read by the tile
    int lo = p.window > 0 ? max(0, pos0 - p.window + 1) : 0;
    lo &= ~(ATC_BN - 1);                                                 // blocks start at multiples of 128 keys
    const int nb = (hi - lo + ATC_BN - 1) / ATC_BN;

    if (warp == 8) {
        // ---------------------------------------------------------------- producer
        // The whole warp: lane l looks up the cache rows of the l-th TMA box of a block (one page
        // or 128 keys), a block ahead of the loads, so that the block-table reads of a block cost
        // one memory latency; lane 0 issues the loads.
        if (lane == 0) {
            mbar_expect_tx(q_full, units * ATC_Q_BYTES);
            for (int u = 0; u < units; ++u) {
                tma_load_2d(tc_smem(sQ) + u * ATC_Q_BYTES, &map_q, q_full, (head0 + u) * ATC_D, tok0);
                tma_load_2d(tc_smem(sQ) + u * ATC_Q_BYTES + ATC_BM * 128, &map_q, q_full, (head0 + u) * ATC_D + 64, tok0);
            }
        }
        const int* table = p.block_table + (int64_t)r * p.table_stride - p.page_base[r];
        const int P = 1 << p.logP;
        const int rows_per_op = P < ATC_BN ? P : ATC_BN;               // rows one TMA box brings
        const int n_ops = ATC_BN / rows_per_op;                          // <= 16 (pages of 8 keys or more)
        const int first_key = p.page_base[r] << p.logP;
        auto row_of = [&](int j) -> int {
            int key = lo + j * ATC_BN + (lane < n_ops ? lane : 0) * rows_per_op;
            // Rows no query of the tile may see (beyond the last query, or in pages a windowed
            // request has given back) are masked later: bring any rows that exist instead.
            if (key >= hi) key = hi - 1 - ((hi - 1) & (rows_per_op - 1));
            if (key < first_key) key = first_key;
            const int page = table[key >> p.logP];
            return ((page * p.nkv + kvh) << p.logP) + (key & (P - 1));
        };
        int slot = 0, phase = 0;
        int row_next = nb > 0 ? row_of(0) : 0;
        bool good = true;
        for (int j = 0; j < nb && good; ++j) {
            const int row_cur = row_next;
            if (j + 1 < nb) row_next = row_of(j + 1);
            for (int kv = 0; kv < 2 && good; ++kv) {                     // the K tile of the block, then its V tile
                bool got = mbar_wait(empty0 + 8 * slot, phase ^ 1);
                if (!got && lane == 0) tc_fail(&g_attn_tc_error, 1, ACORN_KERNEL_ATTN_PREFILL_TC);
                good = __all_sync(0xffffffffu, got);
                if (!good) break;
                if (elect_one()) mbar_expect_tx(full0 + 8 * slot, ATC_TILE_BYTES);
                const uint32_t base = tc_smem(sKV + slot * ATC_TILE_BYTES);
                const CUtensorMap* map = kv ? &map_v : &map_k;
                for (int l = 0; l < n_ops; ++l) {
                    const int row = __shfl_sync(0xffffffffu, row_cur, l);
                    if (elect_one()) {
                        tma_load_2d(base + (uint32_t)(l * rows_per_op) * 128, map, full0 + 8 * slot, 0, row);
                        tma_load_2d(base + ATC_HALF_BYTES + (uint32_t)(l * rows_per_op) * 128, map, full0 + 8 * slot, 64, row);
                    }
                }
                if (++slot == ATC_SLOTS) { slot = 0; phase ^= 1; }
            }
        }
    } else if (warp == 9) {
        // ---------------------------------------------------------------- MMA issuer
        // The whole warp runs this loop, so that its counters, addresses and descriptors are
        // warp-uniform values; one elected lane issues each tcgen05 instruction.
        constexpr uint32_t IDESC_QK = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(ATC_BN >> 3) << 17) |
                                      ((uint32_t)(ATC_BM >> 4) << 24);
        constexpr uint32_t IDESC_PV = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) |
                                      ((uint32_t)(ATC_D >> 3) << 17) | ((uint32_t)(ATC_BM >> 4) << 24);
        auto wait_all = [&](uint32_t bar, uint32_t parity, int code) -> bool {
            bool ok = mbar_wait(bar, parity);
            if (!ok && lane == 0) tc_fail(&g_attn_tc_error, code, ACORN_KERNEL_ATTN_PREFILL_TC);
            return __all_sync(0xffffffffu, ok);
        };
        // descriptor low words (see umma_bf16_lo): Q, and slot 0 as a K tile and as a V tile
        const uint32_t qlo = umma_lo(tc_smem(sQ)), klo0 = umma_lo(tc_smem(sKV));
        const uint32_t vlo0 = umma_lo_mn(tc_smem(sKV), ATC_HALF_BYTES);
        auto issue_qk = [&](int u, int slot) {                          // S_u = Q_u K^T, K in `slot`
            const uint32_t klo = klo0 + slot * (ATC_TILE_BYTES >> 4);
#pragma unroll
            for (int k = 0; k < ATC_D / 16; ++k)
                umma_bf16_elect(tmem_s + u * 128, qlo + ((u * ATC_Q_BYTES + (k >> 2) * ATC_BM * 128) >> 4) + 2 * (k & 3),
                                klo + (((k >> 2) * ATC_HALF_BYTES) >> 4) + 2 * (k & 3), IDESC_QK, k > 0 ? 1u : 0u);
            umma_commit_elect(s_full0 + 8 * u);
        };
        bool good = wait_all(q_full, 0, 2);
        int slot = 0, phase = 0;                                         // the next tile of the ring
        if (good && nb > 0) {
            good = wait_all(full0, 0, 3);
            if (good) {
                for (int u = 0; u < units; ++u) issue_qk(u, 0);
                umma_commit_elect(empty0);
                slot = 1;
            }
        }
        for (int j = 0; j < nb && good; ++j) {
            const int sv = slot, pv = phase;                             // V_j
            if (++slot == ATC_SLOTS) { slot = 0; phase ^= 1; }
            const int sk = slot, pk = phase;                             // K_{j+1}
            const bool has_next = j + 1 < nb;
            if (has_next) { if (++slot == ATC_SLOTS) { slot = 0; phase ^= 1; } }
            good = wait_all(full0 + 8 * sv, pv, 3);
            if (good && has_next) good = wait_all(full0 + 8 * sk, pk, 3);
            if (!good) break;
            const uint32_t vlo = vlo0 + sv * (ATC_TILE_BYTES >> 4);
            for (int u = 0; u < units && good; ++u) {
                good = wait_all(p_full0 + 8 * u, j & 1, 4);
                if (!good) break;
                tc_fence_after();
                // 16 keys a step: P advances 8 columns, V 16 rows of 128 bytes
                umma_bf16_ts_elect(tmem_o + u * 128, tmem_s + u * 128, vlo, IDESC_PV, j > 0 ? 1u : 0u);
#pragma unroll
                for (int k = 1; k < ATC_BN / 16; ++k)
                    umma_bf16_ts_elect(tmem_o + u * 128, tmem_s + u * 128 + 8 * k, vlo + ((k * 16 * 128) >> 4), IDESC_PV, 1u);
                // the next scores go where P was: the pipe runs them after the product above
                if (has_next) issue_qk(u, sk);
                else umma_commit_elect(o_done0 + 8 * u);
            }
            if (!good) break;
            umma_commit_elect(empty0 + 8 * sv);
            if (has_next) umma_commit_elect(empty0 + 8 * sk);
        }
    } else if (warp < 4 * units) {
        // ---------------------------------------------------------------- softmax and output
        const int u = warp >> 2;
        const int row = (warp & 3) * 32 + lane;                          // query row = TMEM lane
        const int head = head0 + u;
        const int qpos = pos0 + row;
        const bool row_ok = row < n_q;
        const uint32_t lane_addr = (uint32_t)((warp & 3) * 32) << 16;
        const uint32_t my_s = tmem_s + lane_addr + u * 128, my_o = tmem_o + lane_addr + u * 128;
        const uint32_t s_full = s_full0 + 8 * u, p_full = p_full0 + 8 * u, o_done = o_done0 + 8 * u;
        float m_ref = -INFINITY, l_run = 0.f;
        bool good = true;
        for (int j = 0; j < nb; ++j) {
            // S of block j is complete; so is P V of block j-1, issued before it: O is stable
            if (good && !mbar_wait(s_full, j & 1)) { tc_fail(&g_attn_tc_error, 6, ACORN_KERNEL_ATTN_PREFILL_TC); good = false; }
            good = __all_sync(0xffffffffu, good);
            if (!good) break;
            tc_fence_after();
            const int key0 = lo + j * ATC_BN;
            // a block every query of the tile sees whole needs no mask
            const bool masked = key0 + ATC_BN - 1 > pos0 || p.window > 0 || n_q < ATC_BM;
            // One pass in the common case: exponentiate against the reference maximum the row
            // already has while the block's own maximum is taken; only a row whose maximum
            // outgrew the reference by more than 2^8 (always so in its first block) moves the
            // reference, and then the warp reads the block again.
            float s[64];
            uint32_t w_lo[32], w_hi[32];
            float neg_ref = m_ref == -INFINITY ? 0.f : -m_ref;
            tmem_ld64(my_s, s);
            if (masked) atc_mask(s, key0, qpos, row_ok, p.window);
            float mx = atc_max(s);
            float psum = atc_exp_pack(s, p.scale_log2, neg_ref, w_lo);
            tmem_ld64(my_s + 64, s);
            if (masked) atc_mask(s, key0 + 64, qpos, row_ok, p.window);
            mx = fmaxf(mx, atc_max(s)) * p.scale_log2;                   // the scale is positive
            float corr = 1.f;
            const bool grew = mx > m_ref + ATC_RESCALE_LOG2;
            if (__any_sync(0xffffffffu, grew)) {
                if (grew) {
                    corr = fast_exp2(m_ref - mx);                        // m_ref = -inf: 0
                    l_run *= corr;
                    m_ref = mx;
                    neg_ref = -m_ref;
                }
                psum = atc_exp_pack(s, p.scale_log2, neg_ref, w_hi);
                tmem_ld64(my_s, s);
                if (masked) atc_mask(s, key0, qpos, row_ok, p.window);
                psum += atc_exp_pack(s, p.scale_log2, neg_ref, w_lo);
            } else {
                psum += atc_exp_pack(s, p.scale_log2, neg_ref, w_hi);
            }
            l_run += psum;
            if (j > 0 && __any_sync(0xffffffffu, corr != 1.f)) {
#pragma unroll
                for (int c = 0; c < ATC_D; c += 32) {
                    float part[32];
                    tmem_ld32(my_o + c, part);
#pragma unroll
                    for (int i = 0; i < 32; ++i) part[i] *= corr;
                    tmem_st32(my_o + c, part);
                }
            }
            // P over the first 64 columns of S: column c holds keys 2c and 2c + 1
            tmem_st32_raw(my_s, w_lo);
            tmem_st32_raw(my_s + 32, w_hi);
            tmem_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(p_full);
        }
        if (good && nb > 0) {
            if (!mbar_wait(o_done, 0)) { tc_fail(&g_attn_tc_error, 8, ACORN_KERNEL_ATTN_PREFILL_TC); good = false; }
            good = __all_sync(0xffffffffu, good);
        }
        if (good) {
            tc_fence_after();
            const float inv = row_ok ? 1.f / l_run : 0.f;
            bf16* orow = p.out + ((int64_t)(tok0 + row) * p.nq + head) * ATC_D;
#pragma unroll
            for (int c = 0; c < ATC_D; c += 32) {
                float part[32];
                tmem_ld32(my_o + c, part);
                if (row_ok) {
#pragma unroll
                    for (int i = 0; i < 32; i += 8) {
                        uint32_t ww[4];
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            __nv_bfloat162 v = __floats2bfloat162_rn(part[i + 2 * q] * inv, part[i + 2 * q + 1] * inv);
                            ww[q] = *reinterpret_cast<uint32_t*>(&v);
                        }
                        *reinterpret_cast<uint4*>(orow + c + i) = make_uint4(ww[0], ww[1], ww[2], ww[3]);
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 9) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;"
                     :: "r"(tmem_base), "r"((uint32_t)ATC_TMEM_COLS) : "memory");
    }
}

// What this kernel takes: head size 128, page size a power of two >= 8, bf16.
extern "C" int acorn_attention_prefill_tc_supported(int nq, int nkv, int d, int P) {
    return nkv > 0 && nq % nkv == 0 && nq <= 65535 && d == ATC_D && P >= 8 && (P & (P - 1)) == 0;
}

// q: [tokens, q_stride] bf16 (query heads first); k_pages / v_pages: [pages, nkv, P, 128] bf16.
extern "C" int acorn_attention_prefill_tc(const void* q, int64_t q_stride, int tokens, void* out, const void* k_pages,
                                          const void* v_pages, int64_t num_pages, const int* block_table,
                                          const int* page_base, int table_stride, const int* row_start,
                                          const int* row_pos, const int* tiles, int n_tiles, int nq, int nkv, int d,
                                          int P, float scale, int window, cudaStream_t stream) {
    if (n_tiles <= 0) return 0;
    if (!acorn_attention_prefill_tc_supported(nq, nkv, d, P) || q_stride % 8 != 0 || ((uintptr_t)q & 15))
        return ACORN_ERR_UNSUPPORTED;
    AttnTcParams p;
    p.out = (bf16*)out; p.block_table = block_table; p.page_base = page_base; p.row_start = row_start;
    p.row_pos = row_pos; p.tiles = tiles; p.table_stride = table_stride; p.nq = nq; p.nkv = nkv;
    p.logP = acorn_log2_exact_tc(P); p.window = window; p.scale_log2 = scale * 1.4426950408889634f;
    p.n_tiles = n_tiles; p.pairs = (nq / nkv + 1) / 2;
    const int64_t ctas = (int64_t)n_tiles * nkv * p.pairs;
    if (ctas > 0x7fffffff) return ACORN_ERR_UNSUPPORTED;
    CUtensorMap mq, mk, mv;
    int rc = make_map(&mq, q, tokens, (int64_t)nq * d, q_stride, 64, ATC_BM);
    if (rc) return rc;
    const int box_rows = P < ATC_BN ? P : ATC_BN;
    rc = make_map(&mk, k_pages, num_pages * nkv * P, d, d, 64, box_rows);
    if (rc) return rc;
    rc = make_map(&mv, v_pages, num_pages * nkv * P, d, d, 64, box_rows);
    if (rc) return rc;
    const size_t smem = ATC_SMEM_TILES + ATC_NUM_BARS * 8 + 16;
    static AcornPerDevice configured;
    if (!configured.seen()) {
        cudaError_t e = cudaFuncSetAttribute(attention_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured.mark();
    }
    return acorn_launch(attention_prefill_tc_kernel, dim3((unsigned)ctas), dim3(ATC_THREADS), smem, stream, mq, mk, mv, p);
}

extern "C" int acorn_attention_tc_error() {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_attn_tc_error, sizeof(int)) != cudaSuccess) return -1;
    if (v != 0) cudaMemcpyToSymbol(g_attn_tc_error, &zero, sizeof(int));
    return v;
}

ACORN_ERROR_WORD_SETTER(acorn_attention_tc_set_error_word)
