// Token choice from float32 logits: argmax, and temperature / top-k / top-p sampling
// with a counter-based random number per (seed, counter), one block per row.
//
// Order of processing as in the reference (acorninfer/sampler.py:38-67): divide by the
// temperature; top-k keeps every logit >= the k-th largest; top-p removes, in ascending
// order, the tokens whose cumulative probability stays <= 1 - top_p (the largest token
// always stays); softmax over what is left; draw.  The draw is by inverse CDF in token
// order with u = uniform(seed, counter): the first token whose running sum exceeds
// u * total.  Rows do not interact, so the result does not depend on the batch.
// temperature == 0 selects argmax (lowest index among equal maxima).
// A row with a NaN or an infinite logit yields token -1 (the host raises).
#include "common.cuh"

#define SAMPLE_THREADS 1024

__device__ __forceinline__ unsigned int float_key(float x) {   // order-preserving map to uint
    unsigned int b = __float_as_uint(x);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

__host__ __device__ __forceinline__ unsigned long long splitmix64(unsigned long long z) {
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

// uniform in [0, 1) with 24 bits, from (seed, counter)
__host__ __device__ __forceinline__ float uniform_from(unsigned long long seed, unsigned long long counter) {
    const unsigned long long z = splitmix64(splitmix64(seed) ^ (counter * 0xD1342543DE82EF95ull));
    return (float)(z >> 40) * (1.0f / 16777216.0f);
}

__device__ __forceinline__ unsigned int block_sum_u32(unsigned int v, unsigned int* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    unsigned int t = (lane < (int)(blockDim.x >> 5)) ? scratch[lane] : 0u;
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    return t;
}

__global__ void __launch_bounds__(SAMPLE_THREADS) sample_kernel(
    const float* __restrict__ logits, int64_t ld, int V, const float* __restrict__ temperature,
    const int* __restrict__ top_k, const float* __restrict__ top_p,
    const unsigned long long* __restrict__ seed, const unsigned long long* __restrict__ counter,
    int* __restrict__ token_out, float* __restrict__ logprob_out) {
    __shared__ float fscratch[32];
    __shared__ unsigned int uscratch[32];
    __shared__ float seg_prefix[SAMPLE_THREADS / 32];
    __shared__ int s_found;
    pdl_wait();
    pdl_trigger();
    const int r = blockIdx.x, tid = threadIdx.x;
    const float* x = logits + (int64_t)r * ld;
    const float temp = temperature[r];

    // pass 1: max (first index among equals) and finiteness
    float best = -INFINITY;
    int best_i = 0x7fffffff;
    unsigned int bad = 0;
    for (int i = tid; i < V; i += SAMPLE_THREADS) {
        const float v = x[i];
        if (!(fabsf(v) <= 3.0e38f)) bad = 1;
        if (v > best) { best = v; best_i = i; }
    }
    bad = block_sum_u32(bad, uscratch);
    const float gmax = block_max(best, fscratch);
    unsigned int cand = (best == gmax) ? (unsigned int)best_i : 0x7fffffffu;
    for (int o = 16; o > 0; o >>= 1) cand = min(cand, __shfl_xor_sync(0xffffffffu, cand, o));
    __syncthreads();
    if ((tid & 31) == 0) uscratch[tid >> 5] = cand;
    __syncthreads();
    cand = (tid & 31) < (SAMPLE_THREADS >> 5) ? uscratch[tid & 31] : 0x7fffffffu;
    for (int o = 16; o > 0; o >>= 1) cand = min(cand, __shfl_xor_sync(0xffffffffu, cand, o));
    const int arg = (int)cand;
    if (bad) {
        if (tid == 0) { token_out[r] = -1; if (logprob_out) logprob_out[r] = 0.f; }
        return;
    }
    if (!(temp > 0.f)) {
        if (tid == 0) { token_out[r] = arg; if (logprob_out) logprob_out[r] = 0.f; }
        return;
    }
    const float inv_t = 1.f / temp;
    // keys of the kept set: key >= lo_key
    unsigned int lo_key = 0u;
    int k = top_k[r];
    if (k > 0 && k < V) {
        // largest K with count(key >= K) >= k  ==  key of the k-th largest logit
        unsigned int lo = 0u, hi = 0xffffffffu;
        while (lo < hi) {
            const unsigned int mid = lo + (unsigned int)(((unsigned long long)hi - lo + 1ull) >> 1);
            unsigned int c = 0;
            for (int i = tid; i < V; i += SAMPLE_THREADS) c += (float_key(x[i]) >= mid);
            c = block_sum_u32(c, uscratch);
            if (c >= (unsigned int)k) lo = mid; else hi = mid - 1u;
        }
        lo_key = lo;
    }
    const float p_keep = top_p[r];
    if (p_keep < 1.f) {
        float z = 0.f;
        for (int i = tid; i < V; i += SAMPLE_THREADS)
            if (float_key(x[i]) >= lo_key) z += expf((x[i] - gmax) * inv_t);
        z = block_sum(z, fscratch);
        const float limit = (1.f - p_keep) * z;
        // smallest K with mass(lo_key <= key <= K) > limit
        unsigned int lo = lo_key, hi = float_key(gmax);
        while (lo < hi) {
            const unsigned int mid = lo + ((hi - lo) >> 1);
            float mass = 0.f;
            for (int i = tid; i < V; i += SAMPLE_THREADS) {
                const unsigned int key = float_key(x[i]);
                if (key >= lo_key && key <= mid) mass += expf((x[i] - gmax) * inv_t);
            }
            mass = block_sum(mass, fscratch);
            if (mass > limit) hi = mid; else lo = mid + 1u;
        }
        lo_key = lo;
    }
    // inverse CDF in token order over the kept set; thread tid owns a contiguous segment
    const int seg = (V + SAMPLE_THREADS - 1) / SAMPLE_THREADS;
    const int i0 = min(V, tid * seg), i1 = min(V, i0 + seg);
    float mine = 0.f;
    for (int i = i0; i < i1; ++i)
        if (float_key(x[i]) >= lo_key) mine += expf((x[i] - gmax) * inv_t);
    // exclusive scan of the 1024 segment sums: inside warps, then over warp totals
    float incl = mine;
    for (int o = 1; o < 32; o <<= 1) {
        const float up = __shfl_up_sync(0xffffffffu, incl, o);
        if ((tid & 31) >= o) incl += up;
    }
    if (tid == 0) s_found = -1;
    if ((tid & 31) == 31) seg_prefix[tid >> 5] = incl;
    __syncthreads();
    if (tid < 32) {
        const float wt = seg_prefix[tid];
        float winc = wt;
        for (int o = 1; o < 32; o <<= 1) {
            const float up = __shfl_up_sync(0xffffffffu, winc, o);
            if (tid >= o) winc += up;
        }
        seg_prefix[tid] = winc - wt;          // exclusive prefix of warp totals
        if (tid == 31) fscratch[0] = winc;    // total
    }
    __syncthreads();
    const float total = fscratch[0];
    const float excl = seg_prefix[tid >> 5] + (incl - mine);
    const float target = uniform_from(seed[r], counter[r]) * total;
    if (mine > 0.f && target >= excl && target < excl + mine) {
        float run = excl;
        int pick = -1, last_kept = -1;
        for (int i = i0; i < i1; ++i) {
            if (float_key(x[i]) >= lo_key) {
                run += expf((x[i] - gmax) * inv_t);
                last_kept = i;
                if (run > target) { pick = i; break; }
            }
        }
        if (pick < 0) pick = last_kept;
        atomicMax(&s_found, pick);
    }
    __syncthreads();
    if (tid == 0) {
        int pick = s_found;
        if (pick < 0) pick = arg;      // rounding left the target beyond the last segment
        token_out[r] = pick;
        if (logprob_out) logprob_out[r] = (x[pick] - gmax) * inv_t - logf(total);
    }
}

extern "C" int acorn_sample(const float* logits, int64_t ld, int rows, int V, const float* temperature,
                            const int* top_k, const float* top_p, const unsigned long long* seed,
                            const unsigned long long* counter, int* token_out, float* logprob_out,
                            cudaStream_t stream) {
    if (rows <= 0) return 0;
    return acorn_launch(sample_kernel, dim3(rows), dim3(SAMPLE_THREADS), 0, stream, logits, ld, V, temperature, top_k,
                        top_p, seed, counter, token_out, logprob_out);
}

// Host copy of the generator, for callers that need the same uniforms off the device.
extern "C" float acorn_uniform(unsigned long long seed, unsigned long long counter) {
    return uniform_from(seed, counter);
}
