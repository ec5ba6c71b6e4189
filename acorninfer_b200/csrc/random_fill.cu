// Counter-based random tensors: element i of a tensor is a function of (key, i) alone, computed
// with integer arithmetic and ONE float32 multiplication (and one addition), so the device kernel,
// the host loop below and a NumPy restatement give the same bits.  Used by the random-weights mode:
// a model drawn on the device for a benchmark is the model a folder written on the host holds.
//
//   h0 = splitmix64(key + 2 i), h1 = splitmix64(key + 2 i + 1)           (64-bit wrap-around)
//   S  = sum of the eight 16-bit lanes of h0 and h1                       (0 .. 8 * 65535)
//   z  = float32(S - 4 * 65535) * scale                                   (one rounding)
//   value = offset + z  (one more rounding; skipped when offset == 0), then rounded to the
//   stored type (bfloat16: round to nearest even).
// The sum of eight uniform lanes has standard deviation 65536 * sqrt(2/3) (Irwin-Hall; tails end at
// 4.9 sigma), so scale = sigma / (65536 * sqrt(2/3)) gives N(0, sigma) to within what weights need.
// Integer tables take h0 & 0x7fff.
#include "common.cuh"

#include <cstring>
#include <thread>
#include <vector>

__host__ __device__ __forceinline__ unsigned long long rf_splitmix64(unsigned long long z) {
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

__host__ __device__ __forceinline__ int rf_lane_sum(unsigned long long key, unsigned long long i,
                                                    unsigned long long* first) {
    const unsigned long long h0 = rf_splitmix64(key + 2ull * i), h1 = rf_splitmix64(key + 2ull * i + 1ull);
    *first = h0;
    int s = 0;
#pragma unroll
    for (int l = 0; l < 4; ++l) s += (int)((h0 >> (16 * l)) & 0xFFFFull) + (int)((h1 >> (16 * l)) & 0xFFFFull);
    return s - 4 * 65535;
}

// kind: 0 float32 out, 1 bfloat16 out, 2 int32 table
template <int KIND>
__global__ void __launch_bounds__(256) random_fill_kernel(void* __restrict__ out, int64_t n, unsigned long long key,
                                                          unsigned long long first, float scale, float offset) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    unsigned long long h0;
    const int s = rf_lane_sum(key, first + (unsigned long long)i, &h0);
    if (KIND == 2) {
        reinterpret_cast<int*>(out)[i] = (int)(h0 & 0x7FFFull);
        return;
    }
    float v = __fmul_rn((float)s, scale);          // never contracted into an fma with the addition below
    if (offset != 0.f) v = __fadd_rn(offset, v);
    if (KIND == 0) reinterpret_cast<float*>(out)[i] = v;
    else reinterpret_cast<bf16*>(out)[i] = __float2bfloat16_rn(v);
}

extern "C" int acorn_random_fill(void* out, int64_t n, unsigned long long key, unsigned long long first, float scale,
                                 float offset, int kind, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (n > (int64_t)2147483647 * 256) return ACORN_ERR_UNSUPPORTED;
    const dim3 grid((unsigned)((n + 255) / 256)), block(256);
    if (kind == 0) random_fill_kernel<0><<<grid, block, 0, stream>>>(out, n, key, first, scale, offset);
    else if (kind == 1) random_fill_kernel<1><<<grid, block, 0, stream>>>(out, n, key, first, scale, offset);
    else if (kind == 2) random_fill_kernel<2><<<grid, block, 0, stream>>>(out, n, key, first, scale, offset);
    else return ACORN_ERR_UNSUPPORTED;
    return acorn_launch_status();
}

// bfloat16 from float32, round to nearest even, on the host (finite inputs only reach here)
static inline unsigned short rf_bf16_bits(float v) {
    unsigned int b;
    memcpy(&b, &v, 4);
    b += 0x7FFFu + ((b >> 16) & 1u);
    return (unsigned short)(b >> 16);
}

// The same values written by host threads into host memory (no device needed): elements
// first .. first + n - 1 of the tensor with this key.
extern "C" int acorn_random_fill_host(void* out, int64_t n, unsigned long long key, unsigned long long first,
                                      float scale, float offset, int kind, int threads) {
    if (kind < 0 || kind > 2) return ACORN_ERR_UNSUPPORTED;
    if (threads < 1) threads = 1;
    auto work = [=](int64_t a, int64_t b) {
        for (int64_t i = a; i < b; ++i) {
            unsigned long long h0;
            const int s = rf_lane_sum(key, first + (unsigned long long)i, &h0);
            if (kind == 2) {
                reinterpret_cast<int*>(out)[i] = (int)(h0 & 0x7FFFull);
                continue;
            }
            volatile float prod = (float)s * scale;           // volatile: rounded to float32 before the addition
            float v = prod;
            if (offset != 0.f) {
                volatile float sum = offset + v;
                v = sum;
            }
            if (kind == 0) reinterpret_cast<float*>(out)[i] = v;
            else reinterpret_cast<unsigned short*>(out)[i] = rf_bf16_bits(v);
        }
    };
    if (threads == 1 || n < (int64_t)1 << 16) {
        work(0, n);
        return 0;
    }
    std::vector<std::thread> pool;
    const int64_t per = (n + threads - 1) / threads;
    for (int t = 0; t < threads; ++t) {
        const int64_t a = t * per, b = a + per < n ? a + per : n;
        if (a < b) pool.emplace_back(work, a, b);
    }
    for (auto& th : pool) th.join();
    return 0;
}
