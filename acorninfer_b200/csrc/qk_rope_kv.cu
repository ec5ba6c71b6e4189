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

// The same for the common case (whole head rotated, half pairing, head size 16, 32, 64, 128 or
// 256): a group of d / 8 lanes takes ROPE_HPG consecutive heads of one token, each lane holding
// four rotary pairs (x[4l .. 4l+3], x[d/2 + 4l .. d/2 + 4l+3]) of every head in registers; vector
// loads (all heads first, then the arithmetic) and stores, no shared memory.  The angles depend
// on the token and the lane only, so cos and sin are computed once for the heads of a group.
// ROPE_HPG = 4 for many tokens (fewer sincos), 1 for few (a decode step: more threads, shorter chains).
template <typename T, int G, int ROPE_HPG>
__global__ void qk_rope_kv_vec_kernel(T* __restrict__ qkv, const float* __restrict__ q_w,
                                      const float* __restrict__ k_w, const float* __restrict__ inv_freq,
                                      const int* __restrict__ positions, const int* __restrict__ token_row,
                                      const int* __restrict__ block_table, const int* __restrict__ page_base,
                                      int table_stride, T* __restrict__ k_pages, T* __restrict__ v_pages,
                                      int tokens, int nq, int nkv, int P, float eps, int write_kv) {
    constexpr int D = G * 8, HALF = D / 2;
    pdl_wait();
    pdl_trigger();
    const int heads = write_kv ? (nq + 2 * nkv) : nq;
    const int groups = (heads + ROPE_HPG - 1) / ROPE_HPG;                // head groups per token
    const int64_t item = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) / G;
    const int l = threadIdx.x % G;
    const bool active = item < (int64_t)tokens * groups;
    const int64_t it = active ? item : 0;
    const int t = (int)(it / groups);
    const int h0 = (int)(it - (int64_t)t * groups) * ROPE_HPG;
    T* tok = qkv + (int64_t)t * (nq + 2 * nkv) * D;
    const int pos = positions[t];
    float4 a[ROPE_HPG], b[ROPE_HPG];
#pragma unroll
    for (int i = 0; i < ROPE_HPG; ++i) {
        const int h = min(h0 + i, heads - 1);
        a[i] = Vec4<T>::load(tok + (int64_t)h * D + 4 * l);
        b[i] = Vec4<T>::load(tok + (int64_t)h * D + HALF + 4 * l);
    }
    int64_t page_off = 0;                                                // of this token's slot, in rows of D
    if (h0 + ROPE_HPG > nq && write_kv) {
        const int r = token_row[t];
        const int page = block_table[(int64_t)r * table_stride + (pos / P - page_base[r])];
        page_off = (int64_t)page * nkv * P + (pos % P);
    }
    float s0 = 0.f, c0 = 1.f, s1 = 0.f, c1 = 1.f, s2 = 0.f, c2 = 1.f, s3 = 0.f, c3 = 1.f;
    if (h0 < nq + nkv) {
        const float4 f = *reinterpret_cast<const float4*>(inv_freq + 4 * l);
        sincosf((float)pos * f.x, &s0, &c0);
        sincosf((float)pos * f.y, &s1, &c1);
        sincosf((float)pos * f.z, &s2, &c2);
        sincosf((float)pos * f.w, &s3, &c3);
    }
#pragma unroll
    for (int i = 0; i < ROPE_HPG; ++i) {
        const bool valid = active && h0 + i < heads;
        const int h = min(h0 + i, heads - 1);
        float4 x = a[i], y = b[i];
        T* dst = tok + (int64_t)h * D;                                   // q: in place
        if (h >= nq) {
            const int kvh = (h - nq) % nkv;
            dst = ((h < nq + nkv) ? k_pages : v_pages) + (page_off + (int64_t)kvh * P) * D;
        }
        // the sum of squares is reduced by every lane of the warp, whatever its head is: lanes of
        // one warp hold heads of different kinds
        float ss = x.x * x.x + x.y * x.y + x.z * x.z + x.w * x.w + y.x * y.x + y.y * y.y + y.z * y.z + y.w * y.w;
#pragma unroll
        for (int o = G / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        if (h < nq + nkv) {
            const float* w = (h < nq) ? q_w : k_w;
            if (w) {
                const float inv = rsqrtf(ss / (float)D + eps);
                const float4 wa = *reinterpret_cast<const float4*>(w + 4 * l);
                const float4 wb = *reinterpret_cast<const float4*>(w + HALF + 4 * l);
                x = make_float4(x.x * inv * wa.x, x.y * inv * wa.y, x.z * inv * wa.z, x.w * inv * wa.w);
                y = make_float4(y.x * inv * wb.x, y.y * inv * wb.y, y.z * inv * wb.z, y.w * inv * wb.w);
            }
            const float4 ra = make_float4(x.x * c0 - y.x * s0, x.y * c1 - y.y * s1, x.z * c2 - y.z * s2, x.w * c3 - y.w * s3);
            const float4 rb = make_float4(y.x * c0 + x.x * s0, y.y * c1 + x.y * s1, y.z * c2 + x.z * s2, y.w * c3 + x.w * s3);
            x = ra;
            y = rb;
        }
        if (valid) {
            Vec4<T>::store(dst + 4 * l, x);
            Vec4<T>::store(dst + HALF + 4 * l, y);
        }
    }
}

template <typename T, int G, int ROPE_HPG>
static int launch_rope_vec_hpg(T* qkv, const float* q_w, const float* k_w, const float* inv_freq, const int* positions,
                           const int* token_row, const int* block_table, const int* page_base, int table_stride,
                           T* k_pages, T* v_pages, int tokens, int nq, int nkv, int P, float eps, int write_kv,
                           cudaStream_t stream) {
    const int heads = write_kv ? (nq + 2 * nkv) : nq;
    const int64_t threads = (int64_t)tokens * ((heads + ROPE_HPG - 1) / ROPE_HPG) * G;
    const int64_t blocks = (threads + 255) / 256;
    return acorn_launch(qk_rope_kv_vec_kernel<T, G, ROPE_HPG>, dim3((unsigned)blocks), dim3(256), 0, stream, qkv, q_w,
                        k_w, inv_freq, positions, token_row, block_table, page_base, table_stride, k_pages, v_pages,
                        tokens, nq, nkv, P, eps, write_kv);
}

template <typename T, int G>
static int launch_rope_vec(T* qkv, const float* q_w, const float* k_w, const float* inv_freq, const int* positions,
                           const int* token_row, const int* block_table, const int* page_base, int table_stride,
                           T* k_pages, T* v_pages, int tokens, int nq, int nkv, int P, float eps, int write_kv,
                           cudaStream_t stream) {
    if (tokens > 256)
        return launch_rope_vec_hpg<T, G, 4>(qkv, q_w, k_w, inv_freq, positions, token_row, block_table, page_base,
                                            table_stride, k_pages, v_pages, tokens, nq, nkv, P, eps, write_kv, stream);
    return launch_rope_vec_hpg<T, G, 1>(qkv, q_w, k_w, inv_freq, positions, token_row, block_table, page_base,
                                        table_stride, k_pages, v_pages, tokens, nq, nkv, P, eps, write_kv, stream);
}

extern "C" int acorn_qk_rope_kv(void* qkv, const float* q_w, const float* k_w, const float* inv_freq,
                                const int* positions, const int* token_row, const int* block_table,
                                const int* page_base, int table_stride, void* k_pages, void* v_pages,
                                int tokens, int nq, int nkv, int d, int rot, int pairing, int P,
                                float eps, int write_kv, int dtype, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (d > 1024 || rot > d || (rot & 1)) return ACORN_ERR_UNSUPPORTED;
    if (rot == d && pairing == 0 && (d == 16 || d == 32 || d == 64 || d == 128 || d == 256)) {
#define ROPE_VEC(G)                                                                                                  \
    ACORN_DISPATCH_DTYPE(dtype, T, return (launch_rope_vec<T, G>((T*)qkv, q_w, k_w, inv_freq, positions, token_row,   \
                                                                  block_table, page_base, table_stride, (T*)k_pages,   \
                                                                  (T*)v_pages, tokens, nq, nkv, P, eps, write_kv,      \
                                                                  stream)))
        switch (d) {
            case 16: ROPE_VEC(2); break;
            case 32: ROPE_VEC(4); break;
            case 64: ROPE_VEC(8); break;
            case 128: ROPE_VEC(16); break;
            default: ROPE_VEC(32); break;
        }
#undef ROPE_VEC
    }
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

// cos and sin of position * inv_freq[j] for every token of a step: out[t][j] = cos, out[t][half + j] = sin
// (float32, the accurate sincosf).  One table serves every layer of the step.
__global__ void rope_table_kernel(const int* __restrict__ positions, const float* __restrict__ inv_freq,
                                  float* __restrict__ out, int tokens, int half) {
    pdl_wait();
    pdl_trigger();
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (int64_t)tokens * half) return;
    const int t = (int)(i / half), j = (int)(i - (int64_t)t * half);
    float s, c;
    sincosf((float)positions[t] * inv_freq[j], &s, &c);
    out[(int64_t)t * 2 * half + j] = c;
    out[(int64_t)t * 2 * half + half + j] = s;
}

extern "C" int acorn_rope_table(const int* positions, const float* inv_freq, float* out, int tokens, int half,
                                cudaStream_t stream) {
    if (tokens <= 0 || half <= 0) return 0;
    const int64_t n = (int64_t)tokens * half;
    return acorn_launch(rope_table_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, positions, inv_freq,
                        out, tokens, half);
}
