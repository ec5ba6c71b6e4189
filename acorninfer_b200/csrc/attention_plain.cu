// Paged causal attention, plain kernel: any mix of prompt portions and decoded tokens,
// any head size, float32 arithmetic throughout.  It is the float32 path's attention
// and the reference the faster kernels are checked against.
//
// One block per (token, query head).  The query at absolute position p of row r reads
// keys lo..p, lo = window ? max(0, p - window + 1) : 0, from the pages of its row:
// key j lives in page block_table[r * stride + j / P - page_base[r]], slot j % P,
// cache layout [num_pages, nkv, P, d].  Query head h uses kv head h / (nq / nkv).
// Scores, softmax (online, per chunk of keys) and the weighted sum are float32.
#include "common.cuh"

#define PLAIN_THREADS 128
#define PLAIN_MAX_D 512

template <typename T>
__global__ void attention_plain_kernel(const T* __restrict__ q, int64_t q_stride, T* __restrict__ out,
                                       const T* __restrict__ k_pages, const T* __restrict__ v_pages,
                                       const int* __restrict__ block_table, const int* __restrict__ page_base,
                                       int table_stride, const int* __restrict__ token_row,
                                       const int* __restrict__ positions, int nq, int nkv, int d, int P,
                                       float scale, int window) {
    extern __shared__ float smem[];
    float* qs = smem;                     // [d]
    float* sc = smem + d;                 // [PLAIN_THREADS] scores / probabilities
    __shared__ int pg[PLAIN_THREADS];     // page of each key of the chunk
    __shared__ float scratch[32];

    const int t = blockIdx.x, h = blockIdx.y;
    const int r = token_row[t], pos = positions[t];
    const int kvh = h / (nq / nkv);
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const int* table = block_table + (int64_t)r * table_stride - page_base[r];
    const T* qp = q + (int64_t)t * q_stride + (int64_t)h * d;
    for (int i = threadIdx.x; i < d; i += blockDim.x) qs[i] = to_float(qp[i]) * scale;

    constexpr int NACC = PLAIN_MAX_D / PLAIN_THREADS;
    float acc[NACC];
#pragma unroll
    for (int a = 0; a < NACC; ++a) acc[a] = 0.f;
    float m = -INFINITY, l = 0.f;
    __syncthreads();

    for (int base = lo; base <= pos; base += PLAIN_THREADS) {
        const int j = base + threadIdx.x;
        float s = -INFINITY;
        if (j <= pos) {
            const int page = table[j / P];
            pg[threadIdx.x] = page;
            const T* kp = k_pages + (((int64_t)page * nkv + kvh) * P + (j % P)) * d;
            float dot = 0.f;
            for (int i = 0; i < d; ++i) dot += qs[i] * to_float(kp[i]);
            s = dot;
        }
        const float cmax = block_max(s, scratch);
        const float m_new = fmaxf(m, cmax);
        const float p = (j <= pos) ? expf(s - m_new) : 0.f;
        sc[threadIdx.x] = p;
        const float psum = block_sum(p, scratch);    // contains __syncthreads: sc, pg visible after
        const float corr = expf(m - m_new);          // m = -inf at first chunk: corr = 0, l = 0
        l = l * corr + psum;
        m = m_new;
        const int n = min(PLAIN_THREADS, pos - base + 1);
#pragma unroll
        for (int a = 0; a < NACC; ++a) {
            const int dim = threadIdx.x + a * PLAIN_THREADS;
            if (dim < d) {
                float v = acc[a] * corr;
                for (int jj = 0; jj < n; ++jj) {
                    const T* vp = v_pages + (((int64_t)pg[jj] * nkv + kvh) * P + ((base + jj) % P)) * d;
                    v += sc[jj] * to_float(vp[dim]);
                }
                acc[a] = v;
            }
        }
        __syncthreads();
    }
    T* op = out + ((int64_t)t * nq + h) * d;
#pragma unroll
    for (int a = 0; a < NACC; ++a) {
        const int dim = threadIdx.x + a * PLAIN_THREADS;
        if (dim < d) op[dim] = from_float<T>(acc[a] / l);
    }
}

extern "C" int acorn_attention_plain(const void* q, int64_t q_stride, void* out, const void* k_pages,
                                     const void* v_pages, const int* block_table, const int* page_base,
                                     int table_stride, const int* token_row, const int* positions,
                                     int tokens, int nq, int nkv, int d, int P, float scale, int window,
                                     int dtype, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (d > PLAIN_MAX_D || nq % nkv != 0 || nq > 65535) return ACORN_ERR_UNSUPPORTED;
    const size_t smem = (size_t)(d + PLAIN_THREADS) * sizeof(float);
    dim3 grid(tokens, nq);
    ACORN_DISPATCH_DTYPE(dtype, T, (attention_plain_kernel<T><<<grid, PLAIN_THREADS, smem, stream>>>(
        (const T*)q, q_stride, (T*)out, (const T*)k_pages, (const T*)v_pages, block_table, page_base,
        table_stride, token_row, positions, nq, nkv, d, P, scale, window)));
    return acorn_launch_status();
}
