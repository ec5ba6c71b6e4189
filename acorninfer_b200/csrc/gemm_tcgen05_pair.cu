// out[M, N] = x[M, K] * W[N, K]^T in bfloat16 for many rows (prompts): tcgen05 tensor cores driven by
// pairs of CTAs on neighbouring SMs (cta_group::2), persistent, warp-specialised.
//
// A pair owns a tile of 256 rows of W by 256 tokens.  Each CTA of the pair loads its own half of both
// operands by TMA (128 rows of W, 128 tokens, 64 elements of K a stage: 32 KB a stage a CTA), and one
// thread of the pair's first CTA issues tcgen05.mma for both: M = 256 (128 rows of W in each CTA's
// tensor memory lanes), N = 256 tokens (each CTA's half of them read from its own shared memory),
// K = 16.  Per byte brought into shared memory the pair multiplies twice what a lone CTA with a
// 128 x 128 tile does, which is what a product of this shape is bound by.
//
//   warp 0      producer: TMA loads through a ring of six stages; the bytes of both CTAs are counted on
//               the first CTA's "full" barrier (loads in the .cta_group::2 form, no multicast)
//   warp 1      in the first CTA: issues the products; tcgen05.commit (multicast to both CTAs) frees a
//               stage in both rings and, after a tile's last k-step, hands the accumulator over
//   warps 2-5   epilogue: tensor memory -> registers -> out; two accumulators of 256 columns, so the
//               epilogue of a tile runs under the products of the next one
//
// Tiles are taken round robin (pair p: tiles p, p + pairs, ...), the token tiles of one W tile next
// to one another, so that a W tile comes from DRAM once.  Every wait is bounded and reports through
// the error word; the two CTAs meet at a cluster barrier before either frees its tensor memory.
#include "tcgen05_helpers.cuh"

#define G2_BM 128            // rows of W a CTA
#define G2_BT 128            // tokens a CTA loads (its half of the pair's 256)
#define G2_BK 64
#define G2_STAGES 6
#define G2_THREADS 192
#define G2_A_BYTES (G2_BM * G2_BK * 2)
#define G2_B_BYTES (G2_BT * G2_BK * 2)
#define G2_STAGE_BYTES (G2_A_BYTES + G2_B_BYTES)
#define G2_ACC_COLS 256
#define G2_SMEM ((size_t)G2_STAGES * G2_STAGE_BYTES + (2 * G2_STAGES + 4) * 8 + 16 + 1024)

__device__ int g_gemm_pair_error = 0;

struct G2Params {
    bf16* out;
    int64_t ldo;
    int M, N, K;
    int kblocks, tiles_m, tiles_n;
};

// A wait bounded in time (two seconds: no wait of this kernel is longer than the kernel before it runs);
// false when it gave up.
__device__ __forceinline__ bool mbar_wait_timed(uint32_t bar, uint32_t parity) {
    long long t0 = 0;
    for (uint32_t tries = 0;; ++tries) {
        if (mbar_test(bar, parity)) return true;
        if ((tries & 1023u) == 1023u) {
            long long now;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
            if (t0 == 0) t0 = now;
            else if (now - t0 > 2000000000ll) return false;
        }
    }
}

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

__global__ void __launch_bounds__(G2_THREADS, 1) gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap map_w,
                                                                          const __grid_constant__ CUtensorMap map_x,
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
        for (int a = 0; a < 2; ++a) { mbar_init(acc_full0 + 8 * a, 1); mbar_init(acc_free0 + 8 * a, 8); }
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
            const int w_row = tn * 2 * G2_BM + (int)rank * G2_BM, x_row = tm * 2 * G2_BT + (int)rank * G2_BT;
            for (int kb = 0; kb < p.kblocks; ++kb, ++g) {
                const int s = g % G2_STAGES;
                bool got = mbar_wait_timed(empty0 + 8 * s, ((g / G2_STAGES) & 1) ^ 1);
                if (!got && lane == 0) tc_fail(&g_gemm_pair_error, 1, ACORN_KERNEL_GEMM_PAIR);
                good = __all_sync(0xffffffffu, got);
                if (!good) break;
                if (elect_one()) {
                    const uint32_t bar = cluster_map(full0 + 8 * s, 0);
                    if (rank == 0) mbar_expect_tx(full0 + 8 * s, 2 * G2_STAGE_BYTES);
                    const uint32_t a = tc_smem(smem + s * G2_STAGE_BYTES);
                    tma_load_2d_pair(a, &map_w, bar, kb * G2_BK, w_row);
                    tma_load_2d_pair(a + G2_A_BYTES, &map_x, bar, kb * G2_BK, x_row);
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
                bool got = mbar_wait_timed(acc_free0 + 8 * as, ((i >> 1) & 1) ^ 1);      // both CTAs have read this accumulator
                if (!got && lane == 0) tc_fail(&g_gemm_pair_error, 2, ACORN_KERNEL_GEMM_PAIR);
                good = __all_sync(0xffffffffu, got);
                if (!good) break;
                tc_fence_after();
                const uint32_t d = tmem_base + (uint32_t)(as * G2_ACC_COLS);
                for (int kb = 0; kb < p.kblocks; ++kb, ++g) {
                    const int s = g % G2_STAGES;
                    got = mbar_wait_timed(full0 + 8 * s, (g / G2_STAGES) & 1);
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
        // ---------------------------------------------------------------- epilogue
        const int quarter = warp & 3;                          // the TMEM lanes this warp may read
        const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
        const uint32_t free_bar0 = cluster_map(acc_free0, 0);
        pdl_wait();
        int i = 0;
        bool good = true;
        for (int tile = pair; tile < tiles && good; tile += pairs, ++i) {
            const int as = i & 1;
            const int tm = tile % p.tiles_m, tn = tile / p.tiles_m;
            const int n = tn * 2 * G2_BM + (int)rank * G2_BM + quarter * 32 + lane;     // this thread's row of W = column of out
            const int m0 = tm * 2 * G2_BT;
            bool got = mbar_wait_timed(acc_full0 + 8 * as, (i >> 1) & 1);
            if (!got && lane == 0) tc_fail(&g_gemm_pair_error, 4, ACORN_KERNEL_GEMM_PAIR);
            good = __all_sync(0xffffffffu, got);
            if (!good) break;
            tc_fence_after();
            const uint32_t taddr = tmem_base + lane_base + (uint32_t)(as * G2_ACC_COLS);
#pragma unroll 1
            for (int c = 0; c < G2_ACC_COLS; c += 32) {
                float v[32];
                tmem_ld32(taddr + c, v);
                if (c + 32 == G2_ACC_COLS) {
                    // the accumulator is in registers: the products of the tile after next may overwrite it
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive_cluster(free_bar0 + 8 * as);
                }
                if (n < p.N) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        const int m = m0 + c + j;
                        if (m < p.M) p.out[(int64_t)m * p.ldo + n] = __float2bfloat16_rn(v[j]);
                    }
                }
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

// What the kernel takes: bf16 operands with K contiguous, K and the row strides multiples of 8 elements,
// 16-byte aligned bases.  It pays from about 128 rows on.
extern "C" int acorn_gemm_tc_pair(const void* x, int64_t ldx, const void* w, int64_t ldw, void* out, int64_t ldo, int M,
                                  int N, int K, int pairs, cudaStream_t stream) {
    if (M < 1 || N < 1 || K < 1 || K % 8 || ldx % 8 || ldw % 8 || pairs < 1) return ACORN_ERR_UNSUPPORTED;
    if (((uintptr_t)x & 15) || ((uintptr_t)w & 15)) return ACORN_ERR_UNSUPPORTED;
    G2Params p = {};
    p.out = (bf16*)out; p.ldo = ldo; p.M = M; p.N = N; p.K = K;
    p.kblocks = (K + G2_BK - 1) / G2_BK;
    p.tiles_m = (M + 2 * G2_BT - 1) / (2 * G2_BT);
    p.tiles_n = (N + 2 * G2_BM - 1) / (2 * G2_BM);
    CUtensorMap mw, mx;
    int rc = make_map(&mw, w, N, K, ldw, G2_BK, G2_BM);
    if (rc) return rc;
    rc = make_map(&mx, x, M, K, ldx, G2_BK, G2_BT);
    if (rc) return rc;
    static AcornPerDevice configured;
    if (!configured.seen()) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)G2_SMEM);
        if (e != cudaSuccess) return (int)e;
        configured.mark();
    }
    const int64_t tiles = (int64_t)p.tiles_m * p.tiles_n;
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
    cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_tcgen05_pair_kernel, mw, mx, p);
    return e != cudaSuccess ? (int)e : acorn_launch_status();
}

// 0, or where a bounded wait gave up since the last call (clears it).
extern "C" int acorn_gemm_tc_pair_error() {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_gemm_pair_error, sizeof(int)) != cudaSuccess) return -1;
    if (v != 0) cudaMemcpyToSymbol(g_gemm_pair_error, &zero, sizeof(int));
    return v;
}

ACORN_ERROR_WORD_SETTER(acorn_gemm_tc_pair_set_error_word)
