// C[M, N] = A[M, K] * W[N, K]^T in true float32: FMA on the CUDA cores, no tensor-core
// mode of reduced precision.  It is the matrix product of the float32 path.  The sum
// over K runs in index order for every output element, so a row's result does not
// depend on M or on the other rows.
//
// A, W: float32 row-major, K contiguous, with row strides lda, ldw; C row stride ldc.
// 64x64 output tile per block, 16-deep K steps, 256 threads with a 4x4 micro-tile each.
#include "common.cuh"

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

extern "C" int acorn_gemm_f32(const float* A, int64_t lda, const float* W, int64_t ldw, float* C,
                              int64_t ldc, int M, int N, int K, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    if (grid.y > 65535) return ACORN_ERR_UNSUPPORTED;
    gemm_f32_kernel<<<grid, 256, 0, stream>>>(A, lda, W, ldw, C, ldc, M, N, K);
    return acorn_launch_status();
}
