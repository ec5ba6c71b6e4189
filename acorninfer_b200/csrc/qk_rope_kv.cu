// Per-head q/k RMSNorm + rotary position encoding + write of K and V into cache pages.
//
// qkv is the projection output [tokens, (nq + 2*nkv) * d]: nq query heads, then nkv
// key heads, then nkv value heads.  For every token and head, in float32:
//   q, k heads:  x <- x * rsqrt(mean(x^2) + eps) * w        (if a norm weight is given)
//                rotate the first `rot` dims by angle pos * inv_freq[j]:
//                  pairing 0 (half):        (x[j], x[j + rot/2])
//                  pairing 1 (interleaved): (x[2j], x[2j+1])
//                  (a, b) <- (a cos - b sin, b cos + a sin)
//   q is written back in place; k goes to the K page, v (untouched) to the V page.
// Cache layout per layer: [num_pages, nkv, page_size, d]; the token at position p of
// row r lives in page block_table[r * table_stride + p / P - page_base[r]], slot p % P.
// With write_kv = 0 only the query heads are processed (a layer that reads another
// layer's cache).
#include "common.cuh"

template <typename T>
__global__ void qk_rope_kv_kernel(T* __restrict__ qkv, const float* __restrict__ q_w,
                                  const float* __restrict__ k_w, const float* __restrict__ inv_freq,
                                  const int* __restrict__ positions, const int* __restrict__ token_row,
                                  const int* __restrict__ block_table, const int* __restrict__ page_base,
                                  int table_stride, T* __restrict__ k_pages, T* __restrict__ v_pages,
                                  int tokens, int nq, int nkv, int d, int rot, int pairing, int P,
                                  float eps, int write_kv) {
    extern __shared__ float smem[];
    pdl_wait();
    pdl_trigger();
    const int warps_per_block = blockDim.x >> 5;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int heads = write_kv ? (nq + 2 * nkv) : nq;
    const int64_t item = (int64_t)blockIdx.x * warps_per_block + warp;
    if (item >= (int64_t)tokens * heads) return;
    const int t = (int)(item / heads);
    const int h = (int)(item - (int64_t)t * heads);
    float* x = smem + warp * d;
    T* src = qkv + ((int64_t)t * (nq + 2 * nkv) + h) * d;
    const int pos = positions[t];

    T* dst = src;   // q: in place
    if (h >= nq) {
        const int r = token_row[t];
        const int kvh = (h - nq) % nkv;
        const int page = block_table[(int64_t)r * table_stride + (pos / P - page_base[r])];
        T* base = (h < nq + nkv) ? k_pages : v_pages;
        dst = base + (((int64_t)page * nkv + kvh) * P + (pos % P)) * d;
    }
    if (h >= nq + nkv) {   // value head: copy
        for (int i = lane; i < d; i += 32) dst[i] = src[i];
        return;
    }
    float ss = 0.f;
    for (int i = lane; i < d; i += 32) {
        const float v = to_float(src[i]);
        x[i] = v;
        ss += v * v;
    }
    const float* w = (h < nq) ? q_w : k_w;
    if (w) {
        ss = warp_sum(ss);
        const float inv = rsqrtf(ss / (float)d + eps);
        __syncwarp();
        for (int i = lane; i < d; i += 32) x[i] = x[i] * inv * w[i];
    }
    __syncwarp();
    const int half = rot >> 1;
    for (int j = lane; j < half; j += 32) {
        const int ia = pairing == 0 ? j : 2 * j;
        const int ib = pairing == 0 ? j + half : 2 * j + 1;
        float s, c;
        sincosf((float)pos * inv_freq[j], &s, &c);
        const float a = x[ia], b = x[ib];
        dst[ia] = from_float<T>(a * c - b * s);
        dst[ib] = from_float<T>(b * c + a * s);
    }
    for (int i = rot + lane; i < d; i += 32) dst[i] = from_float<T>(x[i]);
}

extern "C" int acorn_qk_rope_kv(void* qkv, const float* q_w, const float* k_w, const float* inv_freq,
                                const int* positions, const int* token_row, const int* block_table,
                                const int* page_base, int table_stride, void* k_pages, void* v_pages,
                                int tokens, int nq, int nkv, int d, int rot, int pairing, int P,
                                float eps, int write_kv, int dtype, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (d > 1024 || rot > d || (rot & 1)) return ACORN_ERR_UNSUPPORTED;
    const int warps = 4;
    const int heads = write_kv ? (nq + 2 * nkv) : nq;
    const int64_t items = (int64_t)tokens * heads;
    const int64_t blocks = (items + warps - 1) / warps;
    const size_t smem = (size_t)warps * d * sizeof(float);
    ACORN_DISPATCH_DTYPE(dtype, T, return acorn_launch(
        qk_rope_kv_kernel<T>, dim3((unsigned)blocks), dim3(warps * 32), smem, stream, (T*)qkv, q_w, k_w, inv_freq,
        positions, token_row, block_table, page_base, table_stride, (T*)k_pages, (T*)v_pages, tokens, nq, nkv, d, rot,
        pairing, P, eps, write_kv));
    return ACORN_ERR_UNSUPPORTED;
}
