// Embedding lookup, fused residual-add + RMSNorm, SwiGLU.
#include "common.cuh"

// ---------------------------------------------------------------- embedding
// out32[t, :] = table[ids[t], :]   (float32 residual stream)
template <typename T>
__global__ void embed_kernel(const int* __restrict__ ids, const T* __restrict__ table,
                             float* __restrict__ out32, int H) {
    const int t = blockIdx.x;
    const T* row = table + (int64_t)ids[t] * H;
    float* o = out32 + (int64_t)t * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = to_float(row[i]);
}

extern "C" int acorn_embed(const int* ids, const void* table, float* out32, int tokens, int H,
                           int dtype, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    ACORN_DISPATCH_DTYPE(dtype, T, (embed_kernel<T><<<tokens, 256, 0, stream>>>(ids, (const T*)table, out32, H)));
    return acorn_launch_status();
}

// ---------------------------------------------------------------- add + RMSNorm
// v = resid32[row] (+ delta[row]);  if write_resid: resid32[row] = v
// out[r] = v * rsqrt(mean(v^2) + eps) * w          (all in float32, one rounding)
// row = row_idx ? row_idx[r] : r.  With row_idx the residual is not written back
// (a row may be listed twice).
template <typename T>
__global__ void add_rmsnorm_kernel(float* __restrict__ resid32, const T* __restrict__ delta,
                                   const float* __restrict__ w, T* __restrict__ out,
                                   const int* __restrict__ row_idx, int H, float eps) {
    __shared__ float scratch[32];
    const int r = blockIdx.x;
    const int64_t row = row_idx ? row_idx[r] : r;
    const bool write_resid = (row_idx == nullptr) && (delta != nullptr);
    float* x = resid32 + row * H;
    const T* dl = delta ? delta + row * H : nullptr;
    float ss = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float v = x[i];
        if (dl) v += to_float(dl[i]);
        if (write_resid) x[i] = v;
        ss += v * v;
    }
    ss = block_sum(ss, scratch);
    const float inv = rsqrtf(ss / (float)H + eps);
    T* o = out + (int64_t)r * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float v = x[i];
        if (dl && !write_resid) v += to_float(dl[i]);
        o[i] = from_float<T>(v * inv * w[i]);
    }
}

extern "C" int acorn_add_rmsnorm(float* resid32, const void* delta, const float* w, void* out,
                                 const int* row_idx, int rows, int H, float eps, int dtype,
                                 cudaStream_t stream) {
    if (rows <= 0) return 0;
    const int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
    ACORN_DISPATCH_DTYPE(dtype, T, (add_rmsnorm_kernel<T><<<rows, threads, 0, stream>>>(
        resid32, (const T*)delta, w, (T*)out, row_idx, H, eps)));
    return acorn_launch_status();
}

// ---------------------------------------------------------------- SwiGLU
// out[t, i] = silu(gu[t, i]) * gu[t, I + i],   silu(z) = z / (1 + exp(-z))
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gu, T* __restrict__ out, int64_t total, int I) {
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (int64_t)gridDim.x * blockDim.x) {
        const int64_t t = idx / I;
        const int i = (int)(idx - t * I);
        const float g = to_float(gu[t * 2 * I + i]);
        const float u = to_float(gu[t * 2 * I + I + i]);
        out[idx] = from_float<T>(g / (1.f + expf(-g)) * u);
    }
}

extern "C" int acorn_swiglu(const void* gu, void* out, int tokens, int I, int dtype, cudaStream_t stream) {
    const int64_t total = (int64_t)tokens * I;
    if (total <= 0) return 0;
    int64_t blocks = (total + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    ACORN_DISPATCH_DTYPE(dtype, T, (swiglu_kernel<T><<<(int)blocks, 256, 0, stream>>>(
        (const T*)gu, (T*)out, total, I)));
    return acorn_launch_status();
}

// ---------------------------------------------------------------- casts
template <typename A, typename B>
__global__ void cast_kernel(const A* __restrict__ in, B* __restrict__ out, int64_t n) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
        out[i] = from_float<B>(to_float(in[i]));
}

// dtype_in -> dtype_out over n contiguous elements.
extern "C" int acorn_cast(const void* in, void* out, int64_t n, int dtype_in, int dtype_out, cudaStream_t stream) {
    if (n <= 0) return 0;
    int64_t blocks = (n + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (dtype_in == ACORN_DTYPE_BF16 && dtype_out == ACORN_DTYPE_F32)
        cast_kernel<bf16, float><<<(int)blocks, 256, 0, stream>>>((const bf16*)in, (float*)out, n);
    else if (dtype_in == ACORN_DTYPE_F32 && dtype_out == ACORN_DTYPE_BF16)
        cast_kernel<float, bf16><<<(int)blocks, 256, 0, stream>>>((const float*)in, (bf16*)out, n);
    else
        return ACORN_ERR_UNSUPPORTED;
    return acorn_launch_status();
}
