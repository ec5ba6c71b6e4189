// Paged causal attention, plain kernel: any mix of prompt portions and decoded tokens,
// any head size, float32 arithmetic throughout.  It is the float32 path's attention
// and the reference the faster kernels are checked against.
//
// One block per (token, kv head, up to eight of that kv head's query heads): the query heads of a
// group read the same keys and values, so a key row is fetched once for all of them.  The query at
// absolute position p of row r reads keys lo..p, lo = window ? max(0, p - window + 1) : 0, from
// the pages of its row: key j lives in page block_table[r * stride + j / P - page_base[r]], slot
// j % P, cache layout [num_pages, nkv, P, d].  Query head h uses kv head h / (nq / nkv).
// Scores, softmax (online, per chunk of keys) and the weighted sum are float32.
//
// A chunk is 512 keys.  Scores: one thread a key, the dot products of all the block's query heads
// in one pass over the key row (the rows reach the threads through a hand-over in shared memory, so
// that the loads from the pages are 64 contiguous bytes to four lanes).  Weighted sum: 128 threads across the head's dimensions times four
// groups that take every fourth key; the groups' sums are added at the end.
#include "common.cuh"

#define PLAIN_THREADS 512
#define PLAIN_LANES 128                 // threads across the dimensions of a head
#define PLAIN_KGROUPS (PLAIN_THREADS / PLAIN_LANES)
#define PLAIN_WARPS (PLAIN_THREADS / 32)
#define PLAIN_MAX_D 512
#define PLAIN_HEADS 8                   // query heads a block takes

template <typename T>
__global__ void __launch_bounds__(PLAIN_THREADS) attention_plain_kernel(
    const T* __restrict__ q, int64_t q_stride, T* __restrict__ out, const T* __restrict__ k_pages,
    const T* __restrict__ v_pages, const int* __restrict__ block_table, const int* __restrict__ page_base,
    int table_stride, const int* __restrict__ token_row, const int* __restrict__ positions, int nq, int nkv, int d,
    int P, float scale, int window, int parts) {
    extern __shared__ __align__(16) float smem[];
    float* qs = smem;                                   // [heads][d], scaled
    float* sc = smem + PLAIN_HEADS * d;                 // [heads][PLAIN_THREADS] probabilities of the chunk
    uint4* stage = reinterpret_cast<uint4*>(sc + PLAIN_HEADS * PLAIN_THREADS);   // [warps][32][5] pieces of key rows
    // rows of the pages start on 16-byte boundaries: they can be fetched 16 bytes at a time
    const bool rows_aligned = (d * sizeof(T)) % 16 == 0 && (reinterpret_cast<uintptr_t>(k_pages) & 15) == 0;
    __shared__ int64_t row_at[PLAIN_THREADS];           // where each key of the chunk starts in the pages (keys and values alike)
    __shared__ float red_max[PLAIN_HEADS][PLAIN_WARPS];
    __shared__ float red_sum[PLAIN_HEADS][PLAIN_WARPS];

    const int t = blockIdx.x;
    const int rep = nq / nkv;
    const int kvh = blockIdx.y / parts, part = blockIdx.y % parts;
    const int h0 = kvh * rep + part * PLAIN_HEADS;
    const int G = min(PLAIN_HEADS, rep - part * PLAIN_HEADS);
    const int r = token_row[t], pos = positions[t];
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const int* table = block_table + (int64_t)r * table_stride - page_base[r];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int i = threadIdx.x; i < G * d; i += PLAIN_THREADS)
        qs[i] = to_float(q[(int64_t)t * q_stride + (int64_t)(h0 + i / d) * d + i % d]) * scale;

    constexpr int NACC = PLAIN_MAX_D / PLAIN_LANES;
    const int dlane = threadIdx.x % PLAIN_LANES, kgroup = threadIdx.x / PLAIN_LANES;
    float acc[PLAIN_HEADS][NACC];
    float m[PLAIN_HEADS], l[PLAIN_HEADS];
#pragma unroll
    for (int g = 0; g < PLAIN_HEADS; ++g) {
        m[g] = -INFINITY;
        l[g] = 0.f;
#pragma unroll
        for (int a = 0; a < NACC; ++a) acc[g][a] = 0.f;
    }
    __syncthreads();

    for (int base = lo; base <= pos; base += PLAIN_THREADS) {
        const int j = base + threadIdx.x;
        float s[PLAIN_HEADS];
#pragma unroll
        for (int g = 0; g < PLAIN_HEADS; ++g) s[g] = -INFINITY;
        const bool live = j <= pos;
        int64_t at = 0;
        if (live) at = (((int64_t)table[j / P] * nkv + kvh) * P + (j % P)) * d;
        row_at[threadIdx.x] = at;
        __syncwarp();
        const int wbase = warp * 32;
        const int nlive = min(32, pos - (base + wbase) + 1);            // keys of this warp that exist
        if (nlive > 0) {
            float dot[PLAIN_HEADS];
#pragma unroll
            for (int g = 0; g < PLAIN_HEADS; ++g) dot[g] = 0.f;
            int i = 0;
            if (rows_aligned) {
                // Four 16-byte pieces of every key row at a time.  The warp fetches them together, four
                // neighbouring lanes to a row (64 contiguous bytes), hands them over through shared
                // memory, and every lane then takes the pieces of its own key: the sums run in the
                // order of the elements, as in the loop below.
                constexpr int EPC = 16 / (int)sizeof(T), BATCH = 4 * EPC;
                uint4* mine = stage + wbase * 5;                        // [32 keys][4 pieces + 1]
                for (; i + BATCH <= d; i += BATCH) {
                    uint4 piece[4];
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        const int key = c * 8 + (lane >> 2);
                        piece[c] = make_uint4(0u, 0u, 0u, 0u);
                        if (key < nlive)
                            piece[c] = *reinterpret_cast<const uint4*>(k_pages + row_at[wbase + key] + i + (lane & 3) * EPC);
                    }
#pragma unroll
                    for (int c = 0; c < 4; ++c) mine[(c * 8 + (lane >> 2)) * 5 + (lane & 3)] = piece[c];
                    __syncwarp();
                    uint4 own[4];
#pragma unroll
                    for (int c = 0; c < 4; ++c) own[c] = mine[lane * 5 + c];
                    __syncwarp();
                    const T* kv = reinterpret_cast<const T*>(own);
#pragma unroll
                    for (int u = 0; u < BATCH; u += 4) {
#pragma unroll
                        for (int g = 0; g < PLAIN_HEADS; ++g) {
                            if (g < G) {
                                const float4 q4 = *reinterpret_cast<const float4*>(qs + g * d + i + u);
                                dot[g] += q4.x * to_float(kv[u]);
                                dot[g] += q4.y * to_float(kv[u + 1]);
                                dot[g] += q4.z * to_float(kv[u + 2]);
                                dot[g] += q4.w * to_float(kv[u + 3]);
                            }
                        }
                    }
                }
            }
            if (live) {
                const T* kp = k_pages + at;
                for (; i < d; ++i) {
                    const float kv = to_float(kp[i]);
#pragma unroll
                    for (int g = 0; g < PLAIN_HEADS; ++g)
                        if (g < G) dot[g] += qs[g * d + i] * kv;
                }
#pragma unroll
                for (int g = 0; g < PLAIN_HEADS; ++g)
                    if (g < G) s[g] = dot[g];
            }
        }
#pragma unroll
        for (int g = 0; g < PLAIN_HEADS; ++g) {
            if (g < G) {
                const float w = warp_max(s[g]);
                if (lane == 0) red_max[g][warp] = w;
            }
        }
        __syncthreads();                                 // row_at and the warps' maxima
        float corr[PLAIN_HEADS];
#pragma unroll
        for (int g = 0; g < PLAIN_HEADS; ++g) {
            corr[g] = 1.f;
            if (g < G) {
                float cmax = red_max[g][0];
#pragma unroll
                for (int w = 1; w < PLAIN_WARPS; ++w) cmax = fmaxf(cmax, red_max[g][w]);
                const float m_new = fmaxf(m[g], cmax);
                const float p = (j <= pos) ? expf(s[g] - m_new) : 0.f;
                sc[g * PLAIN_THREADS + threadIdx.x] = p;
                const float ps = warp_sum(p);
                if (lane == 0) red_sum[g][warp] = ps;
                corr[g] = expf(m[g] - m_new);            // m = -inf at the first chunk: corr = 0, l = 0
                m[g] = m_new;
            }
        }
        __syncthreads();                                 // the probabilities and the warps' sums
#pragma unroll
        for (int g = 0; g < PLAIN_HEADS; ++g) {
            if (g < G) {
                float psum = 0.f;
#pragma unroll
                for (int w = 0; w < PLAIN_WARPS; ++w) psum += red_sum[g][w];
                l[g] = l[g] * corr[g] + psum;
#pragma unroll
                for (int a = 0; a < NACC; ++a) acc[g][a] *= corr[g];
            }
        }
        const int n = min(PLAIN_THREADS, pos - base + 1);
        // eight keys at a time: their value elements are asked for together, then added in key order
#pragma unroll
        for (int a = 0; a < NACC; ++a) {
            const int dim = dlane + a * PLAIN_LANES;
            if (a * PLAIN_LANES >= d) break;
            for (int j0 = kgroup; j0 < n; j0 += 8 * PLAIN_KGROUPS) {
                float v[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    const int jj = j0 + u * PLAIN_KGROUPS;
                    v[u] = 0.f;
                    if (jj < n && dim < d)
                        v[u] = to_float(v_pages[row_at[jj] + dim]);
                }
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    const int jj = j0 + u * PLAIN_KGROUPS;
                    if (jj < n) {
#pragma unroll
                        for (int g = 0; g < PLAIN_HEADS; ++g)
                            if (g < G) acc[g][a] += sc[g * PLAIN_THREADS + jj] * v[u];
                    }
                }
            }
        }
        __syncthreads();                                 // sc, row_at and the reduction arrays are free again
    }

    // the key groups' sums, added in the order of the groups, through the probabilities' buffer
    // (heads x 512 floats >= heads x 3 x 128 x dims handled one `a` at a time)
#pragma unroll
    for (int a = 0; a < NACC; ++a) {
        if (a * PLAIN_LANES >= d) break;
#pragma unroll
        for (int g = 0; g < PLAIN_HEADS; ++g)
            if (g < G && kgroup > 0) sc[g * PLAIN_THREADS + (kgroup - 1) * PLAIN_LANES + dlane] = acc[g][a];
        __syncthreads();
        const int dim = dlane + a * PLAIN_LANES;
        if (kgroup == 0 && dim < d) {
#pragma unroll
            for (int g = 0; g < PLAIN_HEADS; ++g) {
                if (g < G) {
                    float v = acc[g][a];
#pragma unroll
                    for (int kg = 1; kg < PLAIN_KGROUPS; ++kg) v += sc[g * PLAIN_THREADS + (kg - 1) * PLAIN_LANES + dlane];
                    out[((int64_t)t * nq + h0 + g) * d + dim] = from_float<T>(v / l[g]);
                }
            }
        }
        __syncthreads();
    }
}

extern "C" int acorn_attention_plain(const void* q, int64_t q_stride, void* out, const void* k_pages,
                                     const void* v_pages, const int* block_table, const int* page_base,
                                     int table_stride, const int* token_row, const int* positions,
                                     int tokens, int nq, int nkv, int d, int P, float scale, int window,
                                     int dtype, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (d < 1 || d > PLAIN_MAX_D || nkv < 1 || nq % nkv != 0) return ACORN_ERR_UNSUPPORTED;
    const int parts = (nq / nkv + PLAIN_HEADS - 1) / PLAIN_HEADS;
    if ((int64_t)nkv * parts > 65535) return ACORN_ERR_UNSUPPORTED;
    // queries and probabilities (at most 32 KB), then the warps' hand-over buffers (40 KB)
    const size_t smem = (size_t)PLAIN_HEADS * (d + PLAIN_THREADS) * sizeof(float) + (size_t)PLAIN_WARPS * 32 * 5 * 16;
    static AcornPerDevice configured;
    if (!configured.seen()) {
        const int most = (int)((size_t)PLAIN_HEADS * (PLAIN_MAX_D + PLAIN_THREADS) * sizeof(float) + (size_t)PLAIN_WARPS * 32 * 5 * 16);
        cudaError_t e = cudaFuncSetAttribute(attention_plain_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, most);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(attention_plain_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, most);
        if (e != cudaSuccess) return (int)e;
        configured.mark();
    }
    dim3 grid(tokens, nkv * parts);
    ACORN_DISPATCH_DTYPE(dtype, T, (attention_plain_kernel<T><<<grid, PLAIN_THREADS, smem, stream>>>(
        (const T*)q, q_stride, (T*)out, (const T*)k_pages, (const T*)v_pages, block_table, page_base,
        table_stride, token_row, positions, nq, nkv, d, P, scale, window, parts)));
    return acorn_launch_status();
}
