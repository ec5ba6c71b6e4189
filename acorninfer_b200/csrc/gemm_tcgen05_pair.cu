// out[M, N] = x[M, K] * W[N, K]^T in bfloat16 for many rows (steps of hundreds to thousands of tokens): tcgen05
// tensor cores driven by pairs of CTAs on neighbouring SMs (cta_group::2), persistent, warp-specialised.
//
// A pair owns a tile of 256 tokens by 256 rows of W.  Each CTA of the pair loads its own half of both
// operands by TMA (128 tokens, 128 rows of W, 64 elements of K a stage: 32 KB a stage a CTA), and one
// thread of the pair's first CTA issues tcgen05.mma for both: M = 256 (128 tokens in each CTA's tensor
// memory lanes), N = 256 rows of W (each CTA's half of them read from its own shared memory), K = 16.
// Per byte brought into shared memory the pair multiplies twice what a lone CTA with a 128 x 128 tile
// does, which is what a product of this shape is bound by.
//
//   warp 0      producer: TMA loads through a ring of six stages; the bytes of both CTAs are counted on
//               the first CTA's "full" barrier (loads in the .cta_group::2 form, no multicast)
//   warp 1      in the first CTA: issues the products; tcgen05.commit (multicast to both CTAs) frees a
//               stage in both rings and, after a tile's last k-step, hands the accumulator over
//   warps 2-9   epilogue: tensor memory -> registers -> memory, two warps to a quarter of the lanes (each
//               takes half of the tile's columns); two accumulators of 256 columns, so the epilogue of a
//               tile runs under the products of the next one
//
// A thread of the epilogue owns one token (its lane of tensor memory) and reads that token's 256
// results of the tile column by column, so everything the epilogues do is local to a thread: a row's
// RMS factor, SwiGLU (gate and up columns of one output), the residual sum with the sum of squares for
// the next norm, a head's RMSNorm and rotation with the write into the cache pages.  A thread stores
// 64 contiguous bytes at a time.
//
// Tiles are taken round robin (pair p: tiles p, p + pairs, ...), the token tiles of one W tile next
// to one another, so that a W tile comes from DRAM once and the pairs that share it read it together.
// (Sharing the work out by k-steps instead, with partial tiles handed over through global memory, was
// built and measured: pairs that run out of step with one another lose the shared reads, and handing
// partial tiles over at the end of a product cost more than the idle SMs of a last, partly filled round.)
// Every wait is bounded and reports through the error word; the two CTAs meet at a cluster barrier
// before either frees its tensor memory.
#include "tcgen05_helpers.cuh"

#define G2_BT 128            // tokens a CTA (lanes of its tensor memory)
#define G2_BW 128            // rows of W a CTA loads (its half of the pair's 256)
#define G2_BK 64
#define G2_STAGES 6
#define G2_THREADS 320
#define G2_A_BYTES (G2_BT * G2_BK * 2)
#define G2_B_BYTES (G2_BW * G2_BK * 2)
#define G2_STAGE_BYTES (G2_A_BYTES + G2_B_BYTES)
#define G2_ACC_COLS 256
#define G2_SMEM ((size_t)G2_STAGES * G2_STAGE_BYTES + (2 * G2_STAGES + 4) * 8 + 16 + 1024)

#define G2_MODE_PLAIN 0       // out = product (bfloat16 or float32)
#define G2_MODE_ADD_NORM 1    // residual += product; out = bf16(residual * norm_w); ss_out = the tile's share of sum(residual^2)
#define G2_MODE_SWIGLU 2      // W in blocks of 64 gate rows + 64 up rows: out = silu(gate) * up, N / 2 columns
#define G2_MODE_QKV_ROPE 3    // W rows are heads of 128: q/k RMSNorm + rotation; k and v to their cache pages

__device__ int g_gemm_pair_error = 0;

struct G2Params {
    void* out;
    int64_t ldo;
    int M, N, K;
    int kblocks, tiles_m, tiles_n;
    int mode, out_f32;
    // rows of x that still lack their factor rsqrt(mean(residual^2) + eps): partial sums of squares
    const float* ss_in;      // [ss_parts, M] or nullptr
    int ss_parts, norm_width;
    float eps;
    // G2_MODE_ADD_NORM
    float* resid;            // [M, ldr] float32, updated in place
    int64_t ldr;
    const float* norm_w;     // [N]
    float* ss_out;           // [2 * tiles_n, M]
    // G2_MODE_QKV_ROPE: nq query heads, nkv key heads, nkv value heads of 128; out takes the query heads
    const int* positions;    // [M]
    const int* token_row;    // [M] row of the block table
    const int* block_table;
    const int* page_base;
    const float* q_w;        // [128] or nullptr: no norm
    const float* k_w;
    const float* inv_freq;   // [64]
    const float* cos_sin;    // [M, 128]: cos then sin of position * inv_freq, or nullptr: computed here
    bf16* k_pages;
    bf16* v_pages;           // nullptr: keys and values are not written
    int table_stride, nq, nkv, logP;
    float rope_eps;
};

__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }

// A TMA tile load whose bytes are counted on a barrier that may lie in the other CTA of the pair.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, uint32_t cluster_bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        :: "r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(cluster_bar), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void umma2_bf16_elect(uint32_t tmem_d, uint32_t alo, uint32_t blo, uint32_t idesc, uint32_t accumulate) {
    if (elect_one()) {
        asm volatile(
            "{\n .reg .pred p;\n .reg .b64 da, db;\n setp.ne.b32 p, %4, 0;\n"
            " mov.b64 da, {%1, %5};\n mov.b64 db, {%2, %5};\n"
            " tcgen05.mma.cta_group::2.kind::f16 [%0], da, db, %3, p;\n}\n"
            :: "r"(tmem_d), "r"(alo), "r"(blo), "r"(idesc), "r"(accumulate), "r"(UMMA_DESC_HI) : "memory");
    }
}
// Arrives on the barrier at this offset in both CTAs of the pair when the products issued so far are done.
__device__ __forceinline__ void umma2_commit_both_elect(uint32_t bar) {
    if (elect_one()) {
        asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                     :: "r"(bar), "h"((uint16_t)3) : "memory");
    }
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_bar) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" :: "r"(cluster_bar) : "memory");
}

// 32 consecutive results of a token, `n_valid` of which exist: to `dst` as bfloat16 (16 bytes at a time when
// the destination allows) or float32.
__device__ __forceinline__ void store_chunk_bf16(bf16* dst, const float (&v)[32], int n_valid) {
    if (n_valid >= 32 && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            uint4 u;
            __nv_bfloat162 t;
            t = __floats2bfloat162_rn(v[8 * q + 0], v[8 * q + 1]); u.x = *reinterpret_cast<uint32_t*>(&t);
            t = __floats2bfloat162_rn(v[8 * q + 2], v[8 * q + 3]); u.y = *reinterpret_cast<uint32_t*>(&t);
            t = __floats2bfloat162_rn(v[8 * q + 4], v[8 * q + 5]); u.z = *reinterpret_cast<uint32_t*>(&t);
            t = __floats2bfloat162_rn(v[8 * q + 6], v[8 * q + 7]); u.w = *reinterpret_cast<uint32_t*>(&t);
            reinterpret_cast<uint4*>(dst)[q] = u;
        }
    } else {
#pragma unroll
        for (int j = 0; j < 32; ++j)
            if (j < n_valid) dst[j] = __float2bfloat16_rn(v[j]);
    }
}
__device__ __forceinline__ void store_chunk_f32(float* dst, const float (&v)[32], int n_valid) {
    if (n_valid >= 32 && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
#pragma unroll
        for (int q = 0; q < 8; ++q)
            reinterpret_cast<float4*>(dst)[q] = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
    } else {
#pragma unroll
        for (int j = 0; j < 32; ++j)
            if (j < n_valid) dst[j] = v[j];
    }
}

__global__ void __launch_bounds__(G2_THREADS, 1) gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap map_x,
                                                                          const __grid_constant__ CUtensorMap map_w,
                                                                          const G2Params p) {
    constexpr uint32_t IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(256 >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (tc_smem(smem_raw) & 1023u)) & 1023u);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + G2_STAGES * G2_STAGE_BYTES);   // full[S], empty[S], acc_full[2], acc_free[2]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * G2_STAGES + 4);
    const uint32_t full0 = tc_smem(bars), empty0 = tc_smem(bars + G2_STAGES);
    const uint32_t acc_full0 = tc_smem(bars + 2 * G2_STAGES), acc_free0 = tc_smem(bars + 2 * G2_STAGES + 2);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_rank();                      // 0: the CTA that issues the products
    const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
    const int tiles = p.tiles_m * p.tiles_n;

    if (threadIdx.x == 0) {
        for (int s = 0; s < G2_STAGES; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(acc_full0 + 8 * a, 1); mbar_init(acc_free0 + 8 * a, 16); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
                     :: "r"(tc_smem(tmem_slot)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    cluster_arrive();                                          // both CTAs' barriers exist before either is signalled from outside
    cluster_wait();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---------------------------------------------------------------- producer
        pdl_wait();
        int g = 0;
        bool good = true;
        for (int tile = pair; tile < tiles && good; tile += pairs) {
            const int tm = tile % p.tiles_m, tn = tile / p.tiles_m;
            const int x_row = tm * 2 * G2_BT + (int)rank * G2_BT, w_row = tn * 2 * G2_BW + (int)rank * G2_BW;
            for (int kb = 0; kb < p.kblocks; ++kb, ++g) {
                const int s = g % G2_STAGES;
                bool got = mbar_wait(empty0 + 8 * s, ((g / G2_STAGES) & 1) ^ 1);
                if (!got && lane == 0) tc_fail(&g_gemm_pair_error, 1, ACORN_KERNEL_GEMM_PAIR);
                good = __all_sync(0xffffffffu, got);
                if (!good) break;
                if (elect_one()) {
                    const uint32_t bar = cluster_map(full0 + 8 * s, 0);
                    if (rank == 0) mbar_expect_tx(full0 + 8 * s, 2 * G2_STAGE_BYTES);
                    const uint32_t a = tc_smem(smem + s * G2_STAGE_BYTES);
                    tma_load_2d_pair(a, &map_x, bar, kb * G2_BK, x_row);
                    tma_load_2d_pair(a + G2_A_BYTES, &map_w, bar, kb * G2_BK, w_row);
                }
            }
        }
        pdl_trigger();
    } else if (warp == 1) {
        // ---------------------------------------------------------------- products (first CTA of the pair)
        if (rank == 0) {
            const uint32_t alo0 = umma_lo(tc_smem(smem)), blo0 = umma_lo(tc_smem(smem) + G2_A_BYTES);
            int g = 0, i = 0;
            bool good = true;
            for (int tile = pair; tile < tiles && good; tile += pairs, ++i) {
                const int as = i & 1;
                bool got = mbar_wait(acc_free0 + 8 * as, ((i >> 1) & 1) ^ 1);      // both CTAs have read this accumulator
                if (!got && lane == 0) tc_fail(&g_gemm_pair_error, 2, ACORN_KERNEL_GEMM_PAIR);
                good = __all_sync(0xffffffffu, got);
                if (!good) break;
                tc_fence_after();
                const uint32_t d = tmem_base + (uint32_t)(as * G2_ACC_COLS);
                for (int kb = 0; kb < p.kblocks; ++kb, ++g) {
                    const int s = g % G2_STAGES;
                    got = mbar_wait(full0 + 8 * s, (g / G2_STAGES) & 1);
                    if (!got && lane == 0) tc_fail(&g_gemm_pair_error, 3, ACORN_KERNEL_GEMM_PAIR);
                    good = __all_sync(0xffffffffu, got);
                    if (!good) break;
                    tc_fence_after();
                    const uint32_t alo = alo0 + s * (G2_STAGE_BYTES >> 4), blo = blo0 + s * (G2_STAGE_BYTES >> 4);
#pragma unroll
                    for (int k = 0; k < G2_BK / 16; ++k)
                        umma2_bf16_elect(d, alo + 2 * k, blo + 2 * k, IDESC, (kb > 0 || k > 0) ? 1u : 0u);
                    umma2_commit_both_elect(empty0 + 8 * s);
                }
                if (good) umma2_commit_both_elect(acc_full0 + 8 * as);
            }
        }
    } else {
        // ---------------------------------------------------------------- epilogue: a thread, a token
        const int quarter = warp & 3;                          // the TMEM lanes this warp may read
        const int half = (warp - 2) >> 2;                      // which 128 of the tile's 256 columns it takes
        const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
        const uint32_t free_bar0 = cluster_map(acc_free0, 0);
        pdl_wait();
        int i = 0;
        bool good = true;
        for (int tile = pair; tile < tiles && good; tile += pairs, ++i) {
            const int as = i & 1;
            const int tm = tile % p.tiles_m, tn = tile / p.tiles_m;
            const int m = tm * 2 * G2_BT + (int)rank * G2_BT + quarter * 32 + lane;      // this thread's token
            const bool m_ok = m < p.M;
            const int n0 = tn * 2 * G2_BW;                                              // first row of W of the tile
            // the token's RMS factor, if its row arrives un-normalised (read while the products run)
            float inv = 1.f;
            if (p.ss_in != nullptr && m_ok) {
                float tot = 0.f;
                for (int q = 0; q < p.ss_parts; ++q) tot += p.ss_in[(int64_t)q * p.M + m];
                inv = rsqrtf(tot / (float)p.norm_width + p.eps);
            }
            bool got = mbar_wait(acc_full0 + 8 * as, (i >> 1) & 1);
            if (!got && lane == 0) tc_fail(&g_gemm_pair_error, 4, ACORN_KERNEL_GEMM_PAIR);
            good = __all_sync(0xffffffffu, got);
            if (!good) break;
            tc_fence_after();
            const uint32_t taddr = tmem_base + lane_base + (uint32_t)(as * G2_ACC_COLS);
            // after the tile's last read of tensor memory: the products of the tile after next may overwrite it
            auto release = [&]() {
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(free_bar0 + 8 * as);
            };
            // 32 columns of this thread's token
            auto load_cols = [&](int c, float (&v)[32]) { tmem_ld32(taddr + c, v); };

            if (p.mode == G2_MODE_PLAIN) {
#pragma unroll 1
                for (int c = half * 128; c < half * 128 + 128; c += 32) {
                    float v[32];
                    load_cols(c, v);
                    if (c + 32 == half * 128 + 128) release();
                    const int nv = p.N - (n0 + c);
                    if (m_ok && nv > 0) {
#pragma unroll
                        for (int j = 0; j < 32; ++j) v[j] *= inv;
                        if (p.out_f32) store_chunk_f32(reinterpret_cast<float*>(p.out) + (int64_t)m * p.ldo + n0 + c, v, nv);
                        else store_chunk_bf16(reinterpret_cast<bf16*>(p.out) + (int64_t)m * p.ldo + n0 + c, v, nv);
                    }
                }
            } else if (p.mode == G2_MODE_SWIGLU) {
                // W rows n0 .. n0 + 255 are two blocks of 64 gate rows and 64 up rows: 128 outputs
                {
                    const int b = half;
#pragma unroll 1
                    for (int c = 0; c < 64; c += 32) {
                        float gt[32], up[32];
                        load_cols(b * 128 + c, gt);
                        load_cols(b * 128 + 64 + c, up);
                        if (c == 32) release();
                        const int oc = tn * 128 + b * 64 + c;
                        const int nv = p.N / 2 - oc;
                        if (m_ok && nv > 0) {
#pragma unroll
                            for (int j = 0; j < 32; ++j) {
                                const float gv = gt[j] * inv, uv = up[j] * inv;
                                gt[j] = gv / (1.f + expf(-gv)) * uv;
                            }
                            store_chunk_bf16(reinterpret_cast<bf16*>(p.out) + (int64_t)m * p.ldo + oc, gt, nv);
                        }
                    }
                }
            } else if (p.mode == G2_MODE_ADD_NORM) {
                float sq = 0.f;
#pragma unroll 1
                for (int c = half * 128; c < half * 128 + 128; c += 32) {
                    float v[32];
                    load_cols(c, v);
                    if (c + 32 == half * 128 + 128) release();
                    const int nv = p.N - (n0 + c);
                    if (m_ok && nv > 0) {
                        float* rp = p.resid + (int64_t)m * p.ldr + n0 + c;
                        const float* wp = p.norm_w + n0 + c;
                        if (nv >= 32 && ((reinterpret_cast<uintptr_t>(rp) | reinterpret_cast<uintptr_t>(wp)) & 15) == 0) {
#pragma unroll
                            for (int q = 0; q < 8; ++q) {
                                const float4 r = reinterpret_cast<const float4*>(rp)[q];
                                v[4 * q] = v[4 * q] * inv + r.x; v[4 * q + 1] = v[4 * q + 1] * inv + r.y;
                                v[4 * q + 2] = v[4 * q + 2] * inv + r.z; v[4 * q + 3] = v[4 * q + 3] * inv + r.w;
                            }
                            store_chunk_f32(rp, v, 32);
#pragma unroll
                            for (int q = 0; q < 8; ++q) {
                                const float4 w = __ldg(reinterpret_cast<const float4*>(wp) + q);
                                sq += v[4 * q] * v[4 * q] + v[4 * q + 1] * v[4 * q + 1] + v[4 * q + 2] * v[4 * q + 2] + v[4 * q + 3] * v[4 * q + 3];
                                v[4 * q] *= w.x; v[4 * q + 1] *= w.y; v[4 * q + 2] *= w.z; v[4 * q + 3] *= w.w;
                            }
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; ++j) {
                                if (j < nv) {
                                    const float r = rp[j] + v[j] * inv;
                                    rp[j] = r;
                                    sq += r * r;
                                    v[j] = r * wp[j];
                                }
                            }
                        }
                        store_chunk_bf16(reinterpret_cast<bf16*>(p.out) + (int64_t)m * p.ldo + n0 + c, v, nv);
                    }
                }
                if (m_ok) p.ss_out[(int64_t)(tn * 2 + half) * p.M + m] = sq;
            } else {
                // G2_MODE_QKV_ROPE: the tile is two heads.  Query and key heads: RMSNorm over the head on the
                // accumulator (float32, no rounding in between), then the rotation of (x[j], x[j + 64]) by
                // position * inv_freq[j]; keys and values go to the token's slot of its cache page.
                const int heads = p.nq + 2 * p.nkv;
                int pos = 0, page = 0;
                if (m_ok) {
                    pos = p.positions[m];
                    if (p.v_pages != nullptr) {
                        const int r = p.token_row[m];
                        page = p.block_table[(int64_t)r * p.table_stride + (pos >> p.logP) - p.page_base[r]];
                    }
                }
                const int hh = half, head = tn * 2 + hh;         // this warp's head of the tile's two
                if (head < heads) {
                    const bool is_q = head < p.nq, is_k = !is_q && head < p.nq + p.nkv;
                    const int kvh = is_q ? 0 : (head - p.nq) % p.nkv;
                    const float* hw = is_q ? p.q_w : is_k ? p.k_w : nullptr;
                    bf16* dst = nullptr;
                    if (m_ok) {
                        if (is_q) dst = reinterpret_cast<bf16*>(p.out) + (int64_t)m * p.ldo + head * 128;
                        else if (p.v_pages != nullptr)
                            dst = (is_k ? p.k_pages : p.v_pages) +
                                  ((((int64_t)page * p.nkv + kvh) << p.logP) + (pos & ((1 << p.logP) - 1))) * 128;
                    }
                    const int th = hh * 128;
                    if (is_q || is_k) {
                        float rinv = 1.f;
                        if (hw != nullptr) {
                            float ss = 0.f;
#pragma unroll 1
                            for (int c = 0; c < 128; c += 32) {
                                float v[32];
                                load_cols(th + c, v);
#pragma unroll
                                for (int j = 0; j < 32; ++j) ss += (v[j] * inv) * (v[j] * inv);
                            }
                            rinv = rsqrtf(ss / 128.f + p.rope_eps);
                        }
#pragma unroll 1
                        for (int c = 0; c < 64; c += 32) {
                            float lo[32], hi[32];
                            load_cols(th + c, lo);
                            load_cols(th + 64 + c, hi);
                            if (dst != nullptr) {
                                const float4* cs4 = p.cos_sin != nullptr
                                    ? reinterpret_cast<const float4*>(p.cos_sin + (int64_t)m * 128 + c) : nullptr;
#pragma unroll
                                for (int j4 = 0; j4 < 32; j4 += 4) {
                                    float cs[4], sn[4];
                                    if (cs4 != nullptr) {
                                        const float4 cc = __ldg(cs4 + j4 / 4), ss4 = __ldg(cs4 + 16 + j4 / 4);
                                        cs[0] = cc.x; cs[1] = cc.y; cs[2] = cc.z; cs[3] = cc.w;
                                        sn[0] = ss4.x; sn[1] = ss4.y; sn[2] = ss4.z; sn[3] = ss4.w;
                                    } else {
#pragma unroll
                                        for (int u = 0; u < 4; ++u) sincosf((float)pos * p.inv_freq[c + j4 + u], &sn[u], &cs[u]);
                                    }
#pragma unroll
                                    for (int u = 0; u < 4; ++u) {
                                        const int j = j4 + u;
                                        const float w1 = hw != nullptr ? hw[c + j] : 1.f, w2 = hw != nullptr ? hw[64 + c + j] : 1.f;
                                        const float x1 = lo[j] * inv * rinv * w1, x2 = hi[j] * inv * rinv * w2;
                                        lo[j] = x1 * cs[u] - x2 * sn[u];
                                        hi[j] = x2 * cs[u] + x1 * sn[u];
                                    }
                                }
                                store_chunk_bf16(dst + c, lo, 32);
                                store_chunk_bf16(dst + 64 + c, hi, 32);
                            }
                        }
                    } else {
#pragma unroll 1
                        for (int c = 0; c < 128; c += 32) {
                            float v[32];
                            load_cols(th + c, v);
                            if (dst != nullptr) {
#pragma unroll
                                for (int j = 0; j < 32; ++j) v[j] *= inv;
                                store_chunk_bf16(dst + c, v, 32);
                            }
                        }
                    }
                }
                release();
            }
        }
    }

    // neither CTA leaves (or frees tensor memory) while the other may still signal its barriers, read its
    // shared memory or wait for its arrivals
    tc_fence_before();
    __syncthreads();
    cluster_arrive();
    cluster_wait();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" :: "r"(tmem_base), "r"(512u) : "memory");
    }
}

// ------------------------------------------------------------------ host side

static int run_pair(const void* x, int64_t ldx, const void* w, int64_t ldw, G2Params& p, int pairs, cudaStream_t stream) {
    const int M = p.M, N = p.N, K = p.K;
    if (M < 1 || N < 1 || K < 1 || K % 8 || ldx % 8 || ldw % 8 || pairs < 1) return ACORN_ERR_UNSUPPORTED;
    if (((uintptr_t)x & 15) || ((uintptr_t)w & 15)) return ACORN_ERR_UNSUPPORTED;
    if (p.ss_in != nullptr && (p.ss_parts < 1 || p.norm_width < 1)) return ACORN_ERR_UNSUPPORTED;
    p.kblocks = (K + G2_BK - 1) / G2_BK;
    p.tiles_m = (M + 2 * G2_BT - 1) / (2 * G2_BT);
    p.tiles_n = (N + 2 * G2_BW - 1) / (2 * G2_BW);
    CUtensorMap mx, mw;
    int rc = make_map(&mx, x, M, K, ldx, G2_BK, G2_BT);
    if (rc) return rc;
    rc = make_map(&mw, w, N, K, ldw, G2_BK, G2_BW);
    if (rc) return rc;
    static AcornPerDevice configured;
    if (!configured.seen()) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)G2_SMEM);
        if (e != cudaSuccess) return (int)e;
        configured.mark();
    }
    const int64_t tiles = (int64_t)p.tiles_m * p.tiles_n;
    if (tiles > 0x3fffffff) return ACORN_ERR_UNSUPPORTED;
    if (pairs > tiles) pairs = (int)tiles;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * pairs);
    cfg.blockDim = dim3(G2_THREADS);
    cfg.dynamicSmemBytes = G2_SMEM;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = acorn_pdl_enabled() ? 2 : 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_tcgen05_pair_kernel, mx, mw, p);
    return e != cudaSuccess ? (int)e : acorn_launch_status();
}

// What the kernel takes: bf16 operands with K contiguous, K and the row strides multiples of 8 elements,
// 16-byte aligned bases; `pairs`: pairs of CTAs to launch (half the device's SMs).  Modes and the ss_in ..
// ss_out arguments as in G2Params.
extern "C" int acorn_gemm_tc_pair(const void* x, int64_t ldx, const void* w, int64_t ldw, void* out, int64_t ldo, int M,
                                  int N, int K, int out_f32, int pairs, int mode, const float* ss_in, int ss_parts,
                                  int norm_width, float eps, float* resid, int64_t ldr, const float* norm_w,
                                  float* ss_out, cudaStream_t stream) {
    if (mode != G2_MODE_PLAIN && mode != G2_MODE_ADD_NORM && mode != G2_MODE_SWIGLU) return ACORN_ERR_UNSUPPORTED;
    if (mode != G2_MODE_PLAIN && out_f32) return ACORN_ERR_UNSUPPORTED;
    if (mode == G2_MODE_SWIGLU && N % 128 != 0) return ACORN_ERR_UNSUPPORTED;
    if (mode == G2_MODE_ADD_NORM && (resid == nullptr || norm_w == nullptr || ss_out == nullptr)) return ACORN_ERR_UNSUPPORTED;
    G2Params p = {};
    p.out = out; p.ldo = ldo; p.M = M; p.N = N; p.K = K; p.out_f32 = out_f32;
    p.mode = mode; p.ss_in = ss_in; p.ss_parts = ss_parts; p.norm_width = norm_width; p.eps = eps;
    p.resid = resid; p.ldr = ldr; p.norm_w = norm_w; p.ss_out = ss_out;
    return run_pair(x, ldx, w, ldw, p, pairs, stream);
}

static inline int g2_log2_exact(int v) {
    if (v <= 0 || (v & (v - 1))) return -1;
    int l = 0;
    while ((1 << l) < v) ++l;
    return l;
}

// The q/k/v product of an attention layer with head size 128 (G2_MODE_QKV_ROPE): w is [(nq + 2 nkv) * 128, K];
// out [M, ldo] takes the query heads; k_pages / v_pages ([pages, nkv, P, 128], P a power of two) the keys
// and values, or nothing when they are nullptr.  cos_sin: [M, 128] float32, cos then sin of position *
// inv_freq for every token (acorn_rope_table), or nullptr: computed in the epilogue.
extern "C" int acorn_gemm_tc_pair_qkv_rope(const void* x, int64_t ldx, const void* w, int64_t ldw, void* out, int64_t ldo,
                                           int M, int K, int pairs, const float* ss_in, int ss_parts, int norm_width,
                                           float eps, const int* positions, const int* token_row, const int* block_table,
                                           const int* page_base, int table_stride, void* k_pages, void* v_pages,
                                           const float* q_w, const float* k_w, const float* inv_freq, const float* cos_sin,
                                           int nq, int nkv, int P, float rope_eps, cudaStream_t stream) {
    const int logP = g2_log2_exact(P);
    if (nq < 1 || nkv < 1 || logP < 0 || positions == nullptr || inv_freq == nullptr) return ACORN_ERR_UNSUPPORTED;
    if ((k_pages == nullptr) != (v_pages == nullptr)) return ACORN_ERR_UNSUPPORTED;
    if (k_pages != nullptr && (token_row == nullptr || block_table == nullptr || page_base == nullptr)) return ACORN_ERR_UNSUPPORTED;
    G2Params p = {};
    p.out = out; p.ldo = ldo; p.M = M; p.N = (nq + 2 * nkv) * 128; p.K = K; p.out_f32 = 0;
    p.mode = G2_MODE_QKV_ROPE; p.ss_in = ss_in; p.ss_parts = ss_parts; p.norm_width = norm_width; p.eps = eps;
    p.positions = positions; p.token_row = token_row; p.block_table = block_table; p.page_base = page_base;
    p.table_stride = table_stride; p.k_pages = (bf16*)k_pages; p.v_pages = (bf16*)v_pages; p.q_w = q_w; p.k_w = k_w;
    p.inv_freq = inv_freq; p.cos_sin = cos_sin; p.nq = nq; p.nkv = nkv; p.logP = logP; p.rope_eps = rope_eps;
    if (cos_sin != nullptr && ((uintptr_t)cos_sin & 15)) return ACORN_ERR_UNSUPPORTED;
    return run_pair(x, ldx, w, ldw, p, pairs, stream);
}

// 0, or where a bounded wait gave up since the last call (clears it).
extern "C" int acorn_gemm_tc_pair_error() {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_gemm_pair_error, sizeof(int)) != cudaSuccess) return -1;
    if (v != 0) cudaMemcpyToSymbol(g_gemm_pair_error, &zero, sizeof(int));
    return v;
}

ACORN_ERROR_WORD_SETTER(acorn_gemm_tc_pair_set_error_word)
