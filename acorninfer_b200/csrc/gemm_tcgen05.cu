// out[M, N] = x[M, K] * W[N, K]^T in bfloat16 on the 5th-generation tensor cores (tcgen05),
// operands staged by TMA, accumulators in tensor memory.
//
// The weight matrix takes the 128-row side of the MMA ("swap-AB"): a CTA owns 128 rows of W
// (output columns n0 .. n0+127) and MB tokens (MB = 16 .. 256), so that a decode step with few
// tokens still fills the instruction and the kernel streams W once at memory speed.  Per
// 64-element step along K, TMA brings a [128 x 64] tile of W and a [MB x 64] tile of x into a
// ring of shared-memory stages (128-byte swizzle, K-major); one elected thread issues four
// tcgen05.mma (M=128, N=MB, K=16) per stage into a [128 lanes x MB columns] float32 accumulator
// in tensor memory; tcgen05.commit frees the stage.  When the K range is split (SPLITS > 1, tiles
// of up to 64 tokens) the CTAs of one output tile form a thread-block cluster, each reduces its
// share of K, and the partial tiles are exchanged by rows through distributed shared memory:
// every CTA reads its accumulator with tcgen05.ld (lane = output column) and stores each row
// into the CTA that finishes it, which adds the partial rows in rank order (deterministic, no
// scratch in global memory, one cluster barrier) and writes out[m, n] as bfloat16 or float32.
//
// The kernel is launched with programmatic stream serialization: the weight tiles of the first
// stages are requested before griddepcontrol.wait, so the weights start to stream while the
// kernel before this one finishes; everything that depends on earlier kernels comes after it.
//
// Every wait on an mbarrier is bounded: when a wait gives up, the kernel records where in
// g_gemm_tc_error, skips the rest of its work, still frees its tensor memory and returns.
#include <cooperative_groups.h>

#include "tcgen05_helpers.cuh"

namespace cg = cooperative_groups;

#define TC_BM 128            // rows of W per CTA (MMA M)
#define TC_BK 64             // elements of K per stage (one 128-byte swizzle row)
#define TC_THREADS 128

__device__ int g_gemm_tc_error = 0;

#define TC_MODE_PLAIN 0       // out = product
#define TC_MODE_ADD_NORM 1    // residual += product; out = bf16(residual * norm_w); ss_out = partial sum of squares
#define TC_MODE_SWIGLU 2      // tiles of 64 gate + 64 up columns: out = silu(gate) * up
#define TC_MODE_QKV_ROPE 3    // tiles are heads of 128: q/k RMSNorm + rotation; k and v to their cache pages
// reduction scratch of the epilogues (floats): four partial sums a row, or a head and its partial sums
#define TC_RED_FLOATS(MB) (4 * (MB) > 256 ? 4 * (MB) : 256)

struct TcParams {
    void* out;
    int64_t ldo;
    int M, N, K;
    int kblocks;             // ceil(K / 64)
    int out_f32;
    int mode;
    // rows of x that still lack their factor rsqrt(mean(residual^2) + eps): partial sums of squares
    const float* ss_in;      // [ss_parts, M] or nullptr
    int ss_parts, norm_width;
    float eps;
    // TC_MODE_ADD_NORM
    float* resid;            // [M, ldr] float32, updated in place
    int64_t ldr;
    const float* norm_w;     // [N]
    float* ss_out;           // [ceil(N / 128), M]
    // TC_MODE_QKV_ROPE: W rows are nq query heads, nkv key heads, nkv value heads of 128; out takes
    // the query heads (row stride ldo), the cache pages [page, nkv, P, 128] the others
    const int* positions;    // [M]
    const int* token_row;    // [M] row of the block table
    const int* block_table;
    const int* page_base;
    const float* q_w;        // [128] or nullptr: no norm
    const float* k_w;
    const float* inv_freq;   // [64]
    bf16* k_pages;
    bf16* v_pages;           // nullptr: keys and values are not written (a layer that reads another's cache)
    int table_stride, nq, nkv, logP;
    float rope_eps;
};

// A load that the compiler leaves where it is written (it may not sink it below a barrier to the
// first use of the value).
__device__ __forceinline__ float ld_global_now(const float* p) {
    float v;
    asm volatile("ld.global.f32 %0, [%1];" : "=f"(v) : "l"(p) : "memory");
    return v;
}

// ------------------------------------------------------------------ the kernel

template <int MB, int STAGES>
__global__ void __launch_bounds__(TC_THREADS) gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_w,
                                                                  const __grid_constant__ CUtensorMap map_x,
                                                                  const TcParams p) {
    constexpr int A_BYTES = TC_BM * TC_BK * 2;           // 16 KB
    constexpr int B_BYTES = MB * TC_BK * 2;
    constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    constexpr int TMEM_COLS = MB < 32 ? 32 : MB;         // power of two >= 32 (MB is 16, 32, 64, 128 or 256)
    constexpr uint32_t IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(MB >> 3) << 17) |
                               ((uint32_t)(TC_BM >> 4) << 24);

    extern __shared__ uint8_t smem_raw[];
    // swizzled tiles need 1024-byte alignment
    uint8_t* smem = smem_raw + ((1024u - (tc_smem(smem_raw) & 1023u)) & 1023u);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);   // full[S], empty[S], accum
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 1);
    const uint32_t full0 = tc_smem(bars), empty0 = tc_smem(bars + STAGES), accum_bar = tc_smem(bars + 2 * STAGES);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = blockIdx.x * TC_BM, m0 = blockIdx.y * MB;
    const int splits = gridDim.z, split = blockIdx.z;
    const int kb0 = (int)((int64_t)p.kblocks * split / splits), kb1 = (int)((int64_t)p.kblocks * (split + 1) / splits);
    const int nkb = kb1 - kb0;

    // Where the receive buffer of the epilogue lies: beside the ring for tiles of up to 32 tokens, in
    // the drained ring for larger ones (which buys them a deeper ring or a third CTA to the SM).
    constexpr bool RECV_IN_RING = MB > 32;
    // every CTA of the cluster says that it runs (or, with the buffer in the ring, that its ring is
    // drained); the epilogue waits for all of them to have said so before it writes into their
    // shared memory
    if (splits > 1 && !RECV_IN_RING) cg::this_cluster().barrier_arrive();
    const int pre = nkb < STAGES ? nkb : STAGES;
    if (warp == 0) {
        // Barriers, then at once the weight tiles of the first stages: they do not depend on the
        // kernel before this one, so they are requested before pdl_wait() and before the rest of
        // the CTA has set itself up; the weights stream while the previous kernel drains.
        if (lane == 0) {
            for (int s = 0; s < STAGES; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
            mbar_init(accum_bar, 1);
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        }
        __syncwarp();
        for (int i = 0; i < pre; ++i) {
            if (elect_one()) {
                mbar_expect_tx(full0 + 8 * i, STAGE_BYTES);
                tma_load_2d(tc_smem(smem + i * STAGE_BYTES), &map_w, full0 + 8 * i, (kb0 + i) * TC_BK, n0);
            }
        }
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     :: "r"(tc_smem(tmem_slot)), "r"((uint32_t)TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;
    bool ok = true;

    if (warp == 0) {
        // ---- producer: the token tiles of the first stages and every later stage come after the
        // wait (the warp stays converged, an elected lane issues)
        pdl_wait();
        for (int i = 0; i < pre; ++i)
            if (elect_one())
                tma_load_2d(tc_smem(smem + i * STAGE_BYTES) + A_BYTES, &map_x, full0 + 8 * i, (kb0 + i) * TC_BK, m0);
        for (int i = pre; i < nkb; ++i) {
            const int s = i % STAGES;
            bool got = mbar_wait(empty0 + 8 * s, ((i / STAGES) & 1) ^ 1);
            if (!got && lane == 0) tc_fail(&g_gemm_tc_error, 1, ACORN_KERNEL_GEMM_TC);
            if (!__all_sync(0xffffffffu, got)) break;
            if (elect_one()) {
                mbar_expect_tx(full0 + 8 * s, STAGE_BYTES);
                const uint32_t a = tc_smem(smem + s * STAGE_BYTES);
                tma_load_2d(a, &map_w, full0 + 8 * s, (kb0 + i) * TC_BK, n0);
                tma_load_2d(a + A_BYTES, &map_x, full0 + 8 * s, (kb0 + i) * TC_BK, m0);
            }
        }
    } else if (warp == 1) {
        // ---- MMA issuer: the whole warp runs the loop (uniform counters and descriptors), one
        // elected lane issues each tcgen05 instruction
        const uint32_t alo0 = umma_lo(tc_smem(smem)), blo0 = umma_lo(tc_smem(smem) + A_BYTES);
        for (int i = 0; i < nkb; ++i) {
            const int s = i % STAGES;
            bool got = mbar_wait(full0 + 8 * s, (i / STAGES) & 1);
            if (!got && lane == 0) tc_fail(&g_gemm_tc_error, 2, ACORN_KERNEL_GEMM_TC);
            if (!__all_sync(0xffffffffu, got)) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t alo = alo0 + s * (STAGE_BYTES >> 4), blo = blo0 + s * (STAGE_BYTES >> 4);
#pragma unroll
            for (int k = 0; k < TC_BK / 16; ++k)     // 16 elements = 32 bytes = 2 descriptor units along K
                umma_bf16_elect(tmem_base, alo + 2 * k, blo + 2 * k, IDESC, (i > 0 || k > 0) ? 1u : 0u);
            umma_commit_elect(empty0 + 8 * s);       // the stage is free once these MMAs have read it
        }
        umma_commit_elect(accum_bar);                // the accumulator is complete
    }
    __syncwarp();

    // ---- epilogue: all four warps; warp w reads TMEM lanes 32w .. 32w+31 (output column n0 + 32w + lane)
    pdl_wait();          // the output buffer may still be read by the kernel before this one
    pdl_trigger();
    if (nkb > 0) ok = mbar_wait(accum_bar, 0);
    if (!ok) tc_fail(&g_gemm_tc_error, 3, ACORN_KERNEL_GEMM_TC);
    ok = __all_sync(0xffffffffu, ok);               // tcgen05.ld below is warp-wide
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const int n = n0 + warp * 32 + lane;
    const int m_valid = min(MB, p.M - m0);
    const uint32_t taddr = tmem_base + ((uint32_t)(warp * 32) << 16);

    // The output tile is finished by rows: row m by the CTA of rank m % csize of the cluster (all
    // rows by the one CTA when K is not split).  Every CTA sends its partial rows from tensor
    // memory straight into the receive buffers of their owners (remote shared-memory stores, which
    // do not wait), the cluster meets once, and each CTA adds up, in rank order, the partial rows
    // it received: recv[q][i][128] is row rank + i * csize as computed by rank q.  For tiles of up
    // to 32 tokens the buffer lies outside the ring, because a peer may still be in its main loop
    // when rows arrive; larger tiles use the ring, and a split one says when its ring is drained
    // (its accumulator is complete: every stage has been read).
    constexpr int RED_FLOATS = TC_RED_FLOATS(MB);
    float* red = reinterpret_cast<float*>(bars + 2 * STAGES + 2);     // reduction scratch, then inv[MB]
    float* inv_s = red + RED_FLOATS;
    float* recv = RECV_IN_RING ? reinterpret_cast<float*>(smem) : inv_s + MB;
    int rank = 0, csize = 1;
    if (splits > 1) {
        cg::cluster_group cluster = cg::this_cluster();
        rank = (int)cluster.block_rank();
        csize = (int)cluster.num_blocks();
    }
    const int slots = (MB + csize - 1) / csize;
    if (splits > 1) {
        if (RECV_IN_RING) cg::this_cluster().barrier_arrive();
        cg::this_cluster().barrier_wait();
    }
    {
        const uint32_t mine = tc_smem(recv) + (uint32_t)((rank * slots * TC_BM + warp * 32 + lane) * 4);
        int owner = 0, slot = 0;                                      // of row c + i
#pragma unroll
        for (int c = 0; c < MB; c += 16) {
            float v[16];
            if (ok && nkb > 0) {
                tmem_ld16(taddr + c, v);
            } else {
#pragma unroll
                for (int i = 0; i < 16; ++i) v[i] = 0.f;
            }
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                if (c + i < m_valid) st_cluster_f32(cluster_map(mine + (uint32_t)(slot * TC_BM * 4), owner), v[i]);
                if (++owner == csize) { owner = 0; ++slot; }
            }
        }
    }
    // Rows of x that arrive un-normalised (x = residual * norm weight): the factor
    // rsqrt(mean(residual^2) + eps) of each row is applied to the product here.
    if (p.ss_in != nullptr) {
        // 128 threads: row = t % MB, the partial sums of a row are shared out over 128 / MB threads
        constexpr int G = TC_THREADS / MB;
        const int m = threadIdx.x % MB, g = threadIdx.x / MB;
        float ss = 0.f;
        if (g < G && m0 + m < p.M)
            for (int q = g; q < p.ss_parts; q += G) ss += p.ss_in[(int64_t)q * p.M + m0 + m];
        if (g < G) red[g * MB + m] = ss;
        __syncthreads();
        if (threadIdx.x < MB) {
            float tot = 0.f;
#pragma unroll
            for (int gg = 0; gg < G; ++gg) tot += red[gg * MB + threadIdx.x];
            inv_s[threadIdx.x] = rsqrtf(tot / (float)p.norm_width + p.eps);
        }
    } else if (threadIdx.x < MB) {
        inv_s[threadIdx.x] = 1.f;
    }
    const int col = threadIdx.x;                                      // 128 threads = 128 columns of the tile
    const bool n_ok = n0 + col < p.N;
    // What the ADD_NORM epilogue reads from global memory is requested before the cluster meets,
    // so that it arrives while the CTAs wait for one another.
    constexpr int MAX_ROWS = MB <= 64 ? MB : 1;                       // the host refuses ADD_NORM for larger tiles
    float r_old[MAX_ROWS];
    float nw = 0.f;
    if (p.mode == TC_MODE_ADD_NORM) {
        if (n_ok) nw = ld_global_now(p.norm_w + n0 + col);
#pragma unroll
        for (int i = 0; i < MAX_ROWS; ++i) {
            const int m = rank + i * csize;
            if (m >= m_valid) break;                                  // the rows of this CTA come first
            r_old[i] = n_ok ? ld_global_now(p.resid + (int64_t)(m0 + m) * p.ldr + n0 + col) : 0.f;
        }
    }
    if (splits > 1) cg::this_cluster().sync();
    else __syncthreads();
    // row rank + i * csize, column c: the partial sums in rank order (independent loads)
    auto tile_sum = [&](int i, int c) -> float {
        float v[8];
#pragma unroll
        for (int q = 0; q < 8; ++q) v[q] = q < csize ? recv[(q * slots + i) * TC_BM + c] : 0.f;
        float acc = v[0];
#pragma unroll
        for (int q = 1; q < 8; ++q) acc += v[q];
        return acc;
    };
    if (p.mode == TC_MODE_PLAIN) {
        for (int i = 0, m = rank; m < m_valid; ++i, m += csize) {
            const float val = tile_sum(i, col) * inv_s[m];
            if (n_ok) {
                const int64_t o = (int64_t)(m0 + m) * p.ldo + n0 + col;
                if (p.out_f32) reinterpret_cast<float*>(p.out)[o] = val;
                else reinterpret_cast<bf16*>(p.out)[o] = __float2bfloat16_rn(val);
            }
        }
    } else if (p.mode == TC_MODE_SWIGLU) {
        // the tile holds 64 gate columns, then the 64 up columns of the same outputs
        for (int i = 0, m = rank; m < m_valid; ++i, m += csize) {
            if (col < 64) {
                const float g = tile_sum(i, col) * inv_s[m], u = tile_sum(i, col + 64) * inv_s[m];
                const int oc = blockIdx.x * 64 + col;
                if (oc < p.N / 2)
                    reinterpret_cast<bf16*>(p.out)[(int64_t)(m0 + m) * p.ldo + oc] =
                        __float2bfloat16_rn(g / (1.f + expf(-g)) * u);
            }
        }
    } else if (p.mode == TC_MODE_QKV_ROPE) {
        // The tile is one head.  Query and key heads: RMSNorm over the head (float32, on the
        // accumulator: no rounding in between), then the rotation of (x[j], x[j + 64]) by
        // position * inv_freq[j]; keys and values go to the token's slot of its cache page.
        const int head = blockIdx.x;
        const bool is_q = head < p.nq, is_k = !is_q && head < p.nq + p.nkv;
        const int kvh = is_q ? 0 : (head - p.nq) % p.nkv;
        const float* hw = is_q ? p.q_w : p.k_w;
        const float wcol = ((is_q || is_k) && hw != nullptr) ? hw[col] : 1.f;
        const float freq = p.inv_freq[col & 63];
        float* xch = red;                                             // [4] partial sums, then [128] the head
        for (int i = 0, m = rank; m < m_valid; ++i, m += csize) {
            float val = tile_sum(i, col) * inv_s[m];
            const int t = m0 + m, pos = p.positions[t];
            if (is_q || is_k) {
                if (hw != nullptr) {
                    const float part = warp_sum(val * val);
                    __syncthreads();                                  // the row before has been read
                    if (lane == 0) xch[warp] = part;
                    __syncthreads();
                    val = val * rsqrtf((xch[0] + xch[1] + xch[2] + xch[3]) / (float)TC_BM + p.rope_eps) * wcol;
                } else {
                    __syncthreads();
                }
                xch[4 + col] = val;
                __syncthreads();
                const float other = xch[4 + (col ^ 64)];
                float sn, cs;
                sincosf((float)pos * freq, &sn, &cs);
                val = col < 64 ? val * cs - other * sn : val * cs + other * sn;
            }
            if (is_q) {
                reinterpret_cast<bf16*>(p.out)[(int64_t)t * p.ldo + head * TC_BM + col] = __float2bfloat16_rn(val);
            } else if (p.v_pages != nullptr) {
                const int r = p.token_row[t];
                const int page = p.block_table[(int64_t)r * p.table_stride + (pos >> p.logP) - p.page_base[r]];
                bf16* dst = (is_k ? p.k_pages : p.v_pages) +
                            ((((int64_t)page * p.nkv + kvh) << p.logP) + (pos & ((1 << p.logP) - 1))) * TC_BM + col;
                *dst = __float2bfloat16_rn(val);
            }
        }
    } else {
        // TC_MODE_ADD_NORM: residual += product; out = bf16(residual * norm weight), not yet
        // scaled; this tile's share of sum(residual^2) per row goes to ss_out[tile][row]
        float sq[MAX_ROWS];
#pragma unroll
        for (int i = 0; i < MAX_ROWS; ++i) {
            const int m = rank + i * csize;
            if (m >= m_valid) break;
            sq[i] = 0.f;
            const float val = tile_sum(i, col) * inv_s[m];
            if (n_ok) {
                const float r = r_old[i] + val;
                p.resid[(int64_t)(m0 + m) * p.ldr + n0 + col] = r;
                reinterpret_cast<bf16*>(p.out)[(int64_t)(m0 + m) * p.ldo + n0 + col] = __float2bfloat16_rn(r * nw);
                sq[i] = r * r;
            }
        }
#pragma unroll
        for (int i = 0; i < MAX_ROWS; ++i) {
            if (rank + i * csize >= m_valid) break;
            const float t = warp_sum(sq[i]);
            if (lane == 0) red[warp * MB + i] = t;
        }
        __syncthreads();
        if (threadIdx.x < MAX_ROWS) {
            const int m = rank + threadIdx.x * csize;
            if (m < m_valid)
                p.ss_out[(int64_t)blockIdx.x * p.M + m0 + m] = red[threadIdx.x] + red[MB + threadIdx.x] +
                                                              red[2 * MB + threadIdx.x] + red[3 * MB + threadIdx.x];
        }
    }

    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem_base), "r"((uint32_t)TMEM_COLS)
                     : "memory");
    }
}

// ------------------------------------------------------------------ host side

template <int MB, int STAGES>
static int launch_tc(const CUtensorMap& mw, const CUtensorMap& mx, const TcParams& p, int splits, cudaStream_t stream) {
    constexpr int STAGE_BYTES = TC_BM * TC_BK * 2 + MB * TC_BK * 2;
    const size_t ring = (size_t)STAGES * STAGE_BYTES;
    const size_t part = (size_t)(MB + 8) * TC_BM * sizeof(float);       // the receive buffer, where it lies in the ring
    const size_t recv = MB <= 32 ? (size_t)(MB + 8) * TC_BM * sizeof(float) : 0;      // see the kernel's epilogue
    const size_t smem = (ring > part ? ring : part) + (2 * STAGES + 2) * 8 +
                        (TC_RED_FLOATS(MB) + MB) * sizeof(float) + recv + 1024;
    static AcornPerDevice configured;
    if (!configured.seen()) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_kernel<MB, STAGES>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured.mark();
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((p.N + TC_BM - 1) / TC_BM, (p.M + MB - 1) / MB, splits);
    cfg.blockDim = dim3(TC_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = splits;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = acorn_pdl_enabled() ? 2 : 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_tcgen05_kernel<MB, STAGES>, mw, mx, p);
    return e != cudaSuccess ? (int)e : acorn_launch_status();
}

// What the kernel takes: bf16 operands with K contiguous, K and both row strides multiples of 8
// elements (16 bytes), 16-byte aligned bases, 1 <= splits <= 8.
extern "C" int acorn_gemm_tc_supported(int64_t M, int64_t N, int64_t K, int64_t ldx, int64_t ldw) {
    return M > 0 && N > 0 && K > 0 && K % 8 == 0 && ldx % 8 == 0 && ldw % 8 == 0 && M <= (1 << 30);
}

static int run_tc(const void* x, int64_t ldx, const void* w, int64_t ldw, TcParams& p, int splits, int per_sm,
                  cudaStream_t stream) {
    const int M = p.M, N = p.N, K = p.K;
    if (!acorn_gemm_tc_supported(M, N, K, ldx, ldw) || splits < 1 || splits > 8) return ACORN_ERR_UNSUPPORTED;
    if (((uintptr_t)x & 15) || ((uintptr_t)w & 15)) return ACORN_ERR_UNSUPPORTED;
    if (p.mode != TC_MODE_PLAIN && (M > 64 || p.out_f32)) return ACORN_ERR_UNSUPPORTED;
    if (p.ss_in != nullptr && (M > 64 || p.ss_parts < 1 || p.norm_width < 1)) return ACORN_ERR_UNSUPPORTED;
    p.kblocks = (K + TC_BK - 1) / TC_BK;
    if (splits > p.kblocks) splits = p.kblocks;
    const int mb = M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : 128;
    if (mb > 64) splits = 1;               // K is split only for tiles of up to 64 tokens
    CUtensorMap mw, mx;
    int rc = make_map(&mw, w, N, K, ldw, TC_BK, TC_BM);
    if (rc) return rc;
    rc = make_map(&mx, x, M, K, ldx, TC_BK, mb);
    if (rc) return rc;
    // per_sm: CTAs that fit on an SM together (2 or 3), bought with the depth of the ring; up to 32
    // tokens only.  Three short rings on an SM stream as well as two long ones and balance better
    // when the tiles do not share out evenly over the SMs.
    switch (mb) {
        case 16: return per_sm == 3 ? launch_tc<16, 3>(mw, mx, p, splits, stream) : launch_tc<16, 5>(mw, mx, p, splits, stream);
        case 32: return per_sm == 3 ? launch_tc<32, 2>(mw, mx, p, splits, stream) : launch_tc<32, 4>(mw, mx, p, splits, stream);
        case 64: return per_sm == 3 ? launch_tc<64, 3>(mw, mx, p, splits, stream) : launch_tc<64, 4>(mw, mx, p, splits, stream);
        default: return launch_tc<128, 3>(mw, mx, p, splits, stream);
    }
}

// mode, ss_in .. ss_out: see TcParams.  Modes other than plain, and ss_in, are for at most 64 rows.
extern "C" int acorn_gemm_tc_ex(const void* x, int64_t ldx, const void* w, int64_t ldw, void* out, int64_t ldo, int M,
                                int N, int K, int out_f32, int splits, int per_sm, int mode, const float* ss_in, int ss_parts,
                                int norm_width, float eps, float* resid, int64_t ldr, const float* norm_w,
                                float* ss_out, cudaStream_t stream) {
    if (mode != TC_MODE_PLAIN && mode != TC_MODE_ADD_NORM && mode != TC_MODE_SWIGLU) return ACORN_ERR_UNSUPPORTED;
    if (mode == TC_MODE_SWIGLU && N % 128 != 0) return ACORN_ERR_UNSUPPORTED;
    if (mode == TC_MODE_ADD_NORM && (resid == nullptr || norm_w == nullptr || ss_out == nullptr)) return ACORN_ERR_UNSUPPORTED;
    TcParams p = {};
    p.out = out; p.ldo = ldo; p.M = M; p.N = N; p.K = K; p.out_f32 = out_f32;
    p.mode = mode; p.ss_in = ss_in; p.ss_parts = ss_parts; p.norm_width = norm_width; p.eps = eps;
    p.resid = resid; p.ldr = ldr; p.norm_w = norm_w; p.ss_out = ss_out;
    return run_tc(x, ldx, w, ldw, p, splits, per_sm, stream);
}

// The q/k/v product of an attention layer with head size 128 (TC_MODE_QKV_ROPE): w is [(nq + 2 nkv)
// * 128, K]; out [M, ldo] takes the query heads; k_pages / v_pages ([pages, nkv, P, 128], P a power
// of two) the keys and values, or nothing when they are nullptr.
extern "C" int acorn_gemm_tc_qkv_rope(const void* x, int64_t ldx, const void* w, int64_t ldw, void* out, int64_t ldo,
                                      int M, int K, int splits, int per_sm, const float* ss_in, int ss_parts,
                                      int norm_width, float eps, const int* positions, const int* token_row,
                                      const int* block_table, const int* page_base, int table_stride, void* k_pages,
                                      void* v_pages, const float* q_w, const float* k_w, const float* inv_freq, int nq,
                                      int nkv, int P, float rope_eps, cudaStream_t stream) {
    const int logP = acorn_log2_exact_tc(P);
    if (nq < 1 || nkv < 1 || logP < 0 || positions == nullptr || inv_freq == nullptr) return ACORN_ERR_UNSUPPORTED;
    if ((k_pages == nullptr) != (v_pages == nullptr)) return ACORN_ERR_UNSUPPORTED;
    if (k_pages != nullptr && (token_row == nullptr || block_table == nullptr || page_base == nullptr)) return ACORN_ERR_UNSUPPORTED;
    TcParams p = {};
    p.out = out; p.ldo = ldo; p.M = M; p.N = (nq + 2 * nkv) * TC_BM; p.K = K; p.out_f32 = 0;
    p.mode = TC_MODE_QKV_ROPE; p.ss_in = ss_in; p.ss_parts = ss_parts; p.norm_width = norm_width; p.eps = eps;
    p.positions = positions; p.token_row = token_row; p.block_table = block_table; p.page_base = page_base;
    p.table_stride = table_stride; p.k_pages = (bf16*)k_pages; p.v_pages = (bf16*)v_pages; p.q_w = q_w; p.k_w = k_w;
    p.inv_freq = inv_freq; p.nq = nq; p.nkv = nkv; p.logP = logP; p.rope_eps = rope_eps;
    return run_tc(x, ldx, w, ldw, p, splits, per_sm, stream);
}

extern "C" int acorn_gemm_tc(const void* x, int64_t ldx, const void* w, int64_t ldw, void* out, int64_t ldo, int M,
                             int N, int K, int out_f32, int splits, cudaStream_t stream) {
    return acorn_gemm_tc_ex(x, ldx, w, ldw, out, ldo, M, N, K, out_f32, splits, 2, TC_MODE_PLAIN, nullptr, 0, 0, 0.f,
                            nullptr, 0, nullptr, nullptr, stream);
}

// Reads and clears the flag that a bounded wait sets when it gives up (0 = no error).
extern "C" int acorn_gemm_tc_error() {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_gemm_tc_error, sizeof(int)) != cudaSuccess) return -1;
    if (v != 0) cudaMemcpyToSymbol(g_gemm_tc_error, &zero, sizeof(int));
    return v;
}

ACORN_ERROR_WORD_SETTER(acorn_gemm_tc_set_error_word)
