// C[M, N] = A[M, K] * W[N, K]^T in true float32: FMA on the CUDA cores, no tensor-core
// mode of reduced precision.  It is the matrix product of the float32 path.
//
// Every kernel here computes an output element as one chain acc = fma(a[k], w[k], acc) over
// k = 0, 1, 2, ... from acc = 0, so the result of a row is the same bits whichever kernel ran
// and does not depend on M, on the other rows or on the tile sizes.
//
// A, W: float32 row-major, K contiguous, with row strides lda, ldw; C row stride ldc.
//   rows kernel   up to 64 rows (decode): 16 rows x 32 columns a block, the weight tiles streamed
//                 through a ring of cp.async stages (the product is bound by reading W once);
//   tile kernel   more rows: 128 x 128 a block, 8 x 8 a thread, the next tile fetched into
//                 registers while this one is multiplied;
//   plain kernel  64 x 64 a block, scalar loads: operands that are not 16-byte aligned.
#include "mma_helpers.cuh"

// ------------------------------------------------------------------ plain kernel

#define BM 64
#define BN 64
#define BK 16

__global__ void __launch_bounds__(256) gemm_f32_kernel(const float* __restrict__ A, int64_t lda,
                                                       const float* __restrict__ W, int64_t ldw,
                                                       float* __restrict__ C, int64_t ldc, int M, int N, int K) {
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;   // 16 x 16 threads
    float acc[4][4] = {};
    for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int idx = threadIdx.x + e * 256;
            const int row = idx >> 4, kk = idx & 15;
            const int k = k0 + kk;
            As[kk][row] = (m0 + row < M && k < K) ? A[(int64_t)(m0 + row) * lda + k] : 0.f;
            Ws[kk][row] = (n0 + row < N && k < K) ? W[(int64_t)(n0 + row) * ldw + k] : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float a[4], w[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) w[j] = Ws[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + ty * 4 + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n < N) C[(int64_t)m * ldc + n] = acc[i][j];
        }
    }
}

// ------------------------------------------------------------------ rows kernel

#define RS_BN 32
#define RS_BK 64
#define RS_ROWS 16
#define RS_STAGES 5
#define RS_LD (RS_BK + 4)       // row stride in shared memory: 16-byte reads of 8 neighbouring rows hit 8 banks groups
#define RS_THREADS 128
#define RS_SMEM (RS_STAGES * (RS_BN + RS_ROWS) * RS_LD * sizeof(float))

// Block b works on columns (b / mblocks) * 32 .. and rows (b % mblocks) * 16 ..: the blocks that
// share a weight tile run next to each other and all but the first find it in L2.
__global__ void __launch_bounds__(RS_THREADS) gemm_f32_rows_kernel(const float* __restrict__ A, int64_t lda,
                                                                   const float* __restrict__ W, int64_t ldw,
                                                                   float* __restrict__ C, int64_t ldc, int M, int N,
                                                                   int K, int mblocks) {
    extern __shared__ __align__(16) float rs_smem[];
    float* Ws = rs_smem;                                          // [stages][32][LD]
    float* As = rs_smem + RS_STAGES * RS_BN * RS_LD;              // [stages][16][LD]
    const int n0 = (blockIdx.x / mblocks) * RS_BN, m0 = (blockIdx.x % mblocks) * RS_ROWS;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;      // column of the tile; rows ty * 4 .. + 3
    const int nk = (K + RS_BK - 1) / RS_BK;

    auto load = [&](int stage, int kb) {
        // chunks of 4 floats: 32 x 16 of W (4 a thread), 16 x 16 of A (2 a thread); outside the matrix: zeros
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int c = threadIdx.x + e * RS_THREADS, row = c >> 4, k = kb * RS_BK + (c & 15) * 4;
            const bool valid = n0 + row < N && k < K;
            const float* src = valid ? W + (int64_t)(n0 + row) * ldw + k : W;
            cp_async_16(smem_addr(Ws + (stage * RS_BN + row) * RS_LD + (c & 15) * 4), src, valid);
        }
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const int c = threadIdx.x + e * RS_THREADS, row = c >> 4, k = kb * RS_BK + (c & 15) * 4;
            const bool valid = m0 + row < M && k < K;
            const float* src = valid ? A + (int64_t)(m0 + row) * lda + k : A;
            cp_async_16(smem_addr(As + (stage * RS_ROWS + row) * RS_LD + (c & 15) * 4), src, valid);
        }
    };

    for (int s = 0; s < RS_STAGES - 1; ++s) {
        if (s < nk) load(s, s);
        cp_async_commit();
    }
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (int kb = 0; kb < nk; ++kb) {
        cp_async_wait<RS_STAGES - 2>();          // this thread's copies of stage kb have landed
        __syncthreads();                         // everyone's have, and everyone is done with stage kb - 1
        if (kb + RS_STAGES - 1 < nk) load((kb + RS_STAGES - 1) % RS_STAGES, kb + RS_STAGES - 1);
        cp_async_commit();
        const int stage = kb % RS_STAGES;
        const float* wrow = Ws + (stage * RS_BN + tx) * RS_LD;
        const float* arow = As + (stage * RS_ROWS + ty * 4) * RS_LD;
#pragma unroll 4
        for (int kk = 0; kk < RS_BK; kk += 4) {
            const float4 w = *reinterpret_cast<const float4*>(wrow + kk);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float4 a = *reinterpret_cast<const float4*>(arow + i * RS_LD + kk);
                acc[i] = fmaf(a.x, w.x, acc[i]);
                acc[i] = fmaf(a.y, w.y, acc[i]);
                acc[i] = fmaf(a.z, w.z, acc[i]);
                acc[i] = fmaf(a.w, w.w, acc[i]);
            }
        }
    }
    cp_async_wait<0>();
    if (n0 + tx < N) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int m = m0 + ty * 4 + i;
            if (m < M) C[(int64_t)m * ldc + n0 + tx] = acc[i];
        }
    }
}

// ------------------------------------------------------------------ tile kernel

#define TL_BM 128
#define TL_BN 128
#define TL_BK 16
#define TL_LD (TL_BM + 4)
#define TL_THREADS 256

__global__ void __launch_bounds__(TL_THREADS, 2) gemm_f32_tile_kernel(const float* __restrict__ A, int64_t lda,
                                                                      const float* __restrict__ W, int64_t ldw,
                                                                      float* __restrict__ C, int64_t ldc, int M, int N,
                                                                      int K) {
    __shared__ __align__(16) float As[2][TL_BK][TL_LD];        // transposed: [k][row]
    __shared__ __align__(16) float Ws[2][TL_BK][TL_LD];
    const int m0 = blockIdx.y * TL_BM, n0 = blockIdx.x * TL_BN;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;      // columns tx * 4 .. + 3 and 64 + ..; rows ty * 4 .. likewise
    const int nt = (K + TL_BK - 1) / TL_BK;
    // a tile is 128 rows x 4 chunks of 4 floats: two chunks of A and two of W a thread
    const int lrow = threadIdx.x >> 2, lseg = (threadIdx.x & 3) * 4;
    float4 ra[2], rw[2];

    auto fetch = [&](int t) {
        const int k = t * TL_BK + lseg;
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const int row = lrow + e * 64;
            ra[e] = (m0 + row < M && k < K) ? *reinterpret_cast<const float4*>(A + (int64_t)(m0 + row) * lda + k)
                                            : make_float4(0.f, 0.f, 0.f, 0.f);
            rw[e] = (n0 + row < N && k < K) ? *reinterpret_cast<const float4*>(W + (int64_t)(n0 + row) * ldw + k)
                                            : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    };
    auto stash = [&](int buf) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const int row = lrow + e * 64;
            As[buf][lseg + 0][row] = ra[e].x; As[buf][lseg + 1][row] = ra[e].y;
            As[buf][lseg + 2][row] = ra[e].z; As[buf][lseg + 3][row] = ra[e].w;
            Ws[buf][lseg + 0][row] = rw[e].x; Ws[buf][lseg + 1][row] = rw[e].y;
            Ws[buf][lseg + 2][row] = rw[e].z; Ws[buf][lseg + 3][row] = rw[e].w;
        }
    };

    float acc[8][8];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;
    fetch(0);
    stash(0);
    __syncthreads();
    for (int t = 0; t < nt; ++t) {
        const int buf = t & 1;
        if (t + 1 < nt) fetch(t + 1);            // in flight while this tile is multiplied
#pragma unroll
        for (int kk = 0; kk < TL_BK; ++kk) {
            const float4 a0 = *reinterpret_cast<const float4*>(&As[buf][kk][ty * 4]);
            const float4 a1 = *reinterpret_cast<const float4*>(&As[buf][kk][64 + ty * 4]);
            const float4 w0 = *reinterpret_cast<const float4*>(&Ws[buf][kk][tx * 4]);
            const float4 w1 = *reinterpret_cast<const float4*>(&Ws[buf][kk][64 + tx * 4]);
            const float a[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
            const float w[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
            for (int i = 0; i < 8; ++i)
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
        }
        if (t + 1 < nt) stash(buf ^ 1);          // the other buffer was last read before the barrier below, a tile ago
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int m = m0 + (i < 4 ? ty * 4 + i : 64 + ty * 4 + i - 4);
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int n = n0 + (j < 4 ? tx * 4 + j : 64 + tx * 4 + j - 4);
            if (n < N) C[(int64_t)m * ldc + n] = acc[i][j];
        }
    }
}

// ------------------------------------------------------------------ host side

extern "C" int acorn_gemm_f32(const float* A, int64_t lda, const float* W, int64_t ldw, float* C,
                              int64_t ldc, int M, int N, int K, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    // the faster kernels move 16 bytes at a time along K
    const bool aligned = K % 4 == 0 && lda % 4 == 0 && ldw % 4 == 0 && ((uintptr_t)A & 15) == 0 && ((uintptr_t)W & 15) == 0;
    if (aligned && M <= 64) {
        static AcornPerDevice configured;
        if (!configured.seen()) {
            cudaError_t e = cudaFuncSetAttribute(gemm_f32_rows_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)RS_SMEM);
            if (e != cudaSuccess) return (int)e;
            configured.mark();
        }
        const int mblocks = (M + RS_ROWS - 1) / RS_ROWS;
        const int64_t blocks = (int64_t)((N + RS_BN - 1) / RS_BN) * mblocks;
        if (blocks > 0x7fffffff) return ACORN_ERR_UNSUPPORTED;
        gemm_f32_rows_kernel<<<(unsigned)blocks, RS_THREADS, RS_SMEM, stream>>>(A, lda, W, ldw, C, ldc, M, N, K, mblocks);
        return acorn_launch_status();
    }
    if (aligned) {
        dim3 grid((N + TL_BN - 1) / TL_BN, (M + TL_BM - 1) / TL_BM);
        if (grid.y > 65535) return ACORN_ERR_UNSUPPORTED;
        gemm_f32_tile_kernel<<<grid, TL_THREADS, 0, stream>>>(A, lda, W, ldw, C, ldc, M, N, K);
        return acorn_launch_status();
    }
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    if (grid.y > 65535) return ACORN_ERR_UNSUPPORTED;
    gemm_f32_kernel<<<grid, 256, 0, stream>>>(A, lda, W, ldw, C, ldc, M, N, K);
    return acorn_launch_status();
}
