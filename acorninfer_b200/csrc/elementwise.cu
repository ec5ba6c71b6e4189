// Embedding lookup, fused residual-add + RMSNorm, SwiGLU.
#include "common.cuh"

// ---------------------------------------------------------------- embedding
// out32[t, :] = table[ids[t], :]   (float32 residual stream)
template <typename T>
__global__ void embed_kernel(const int* __restrict__ ids, const T* __restrict__ table,
                             float* __restrict__ out32, int H) {
    pdl_wait();
    pdl_trigger();
    const int t = blockIdx.x;
    const T* row = table + (int64_t)ids[t] * H;
    float* o = out32 + (int64_t)t * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = to_float(row[i]);
}

extern "C" int acorn_embed(const int* ids, const void* table, float* out32, int tokens, int H,
                           int dtype, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    ACORN_DISPATCH_DTYPE(dtype, T, return acorn_launch(embed_kernel<T>, dim3(tokens), dim3(256), 0, stream, ids, (const T*)table, out32, H));
    return ACORN_ERR_UNSUPPORTED;
}

// token_ids[dst[i]] = src_tokens[src[i]]: the ids a step decodes from are the ids the step before it
// sampled, taken on the device (the host reads them one step later).
__global__ void patch_tokens_kernel(int* __restrict__ token_ids, const int* __restrict__ dst,
                                    const int* __restrict__ src, const int* __restrict__ src_tokens, int n) {
    pdl_wait();
    pdl_trigger();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) token_ids[dst[i]] = src_tokens[src[i]];
}

extern "C" int acorn_patch_tokens(int* token_ids, const int* dst, const int* src, const int* src_tokens, int n,
                                  cudaStream_t stream) {
    if (n <= 0) return 0;
    return acorn_launch(patch_tokens_kernel, dim3((n + 127) / 128), dim3(128), 0, stream, token_ids, dst, src,
                        src_tokens, n);
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
    pdl_wait();
    pdl_trigger();
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

// The same with four elements per thread and step, the row kept in registers between the two
// passes: for widths that are a multiple of 4 and at most threads * 4 * RMS_MAX_ITER.
#define RMS_MAX_ITER 8

template <typename T>
__global__ void add_rmsnorm_vec_kernel(float* __restrict__ resid32, const T* __restrict__ delta,
                                       const float* __restrict__ w, T* __restrict__ out,
                                       const int* __restrict__ row_idx, int H, float eps) {
    __shared__ float scratch[32];
    pdl_wait();
    pdl_trigger();
    const int r = blockIdx.x;
    const int64_t row = row_idx ? row_idx[r] : r;
    const bool write_resid = (row_idx == nullptr) && (delta != nullptr);
    float* x = resid32 + row * H;
    const T* dl = delta ? delta + row * H : nullptr;
    float4 v[RMS_MAX_ITER];
    float ss = 0.f;
#pragma unroll
    for (int it = 0; it < RMS_MAX_ITER; ++it) {
        const int i = (it * blockDim.x + threadIdx.x) * 4;
        if (i < H) {
            float4 a = *reinterpret_cast<const float4*>(x + i);
            if (dl) {
                const float4 d = Vec4<T>::load(dl + i);
                a.x += d.x; a.y += d.y; a.z += d.z; a.w += d.w;
            }
            if (write_resid) *reinterpret_cast<float4*>(x + i) = a;
            ss += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
            v[it] = a;
        }
    }
    ss = block_sum(ss, scratch);
    const float inv = rsqrtf(ss / (float)H + eps);
    T* o = out + (int64_t)r * H;
#pragma unroll
    for (int it = 0; it < RMS_MAX_ITER; ++it) {
        const int i = (it * blockDim.x + threadIdx.x) * 4;
        if (i < H) {
            const float4 ww = *reinterpret_cast<const float4*>(w + i);
            Vec4<T>::store(o + i, make_float4(v[it].x * inv * ww.x, v[it].y * inv * ww.y, v[it].z * inv * ww.z,
                                              v[it].w * inv * ww.w));
        }
    }
}

extern "C" int acorn_add_rmsnorm(float* resid32, const void* delta, const float* w, void* out,
                                 const int* row_idx, int rows, int H, float eps, int dtype,
                                 cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (H % 4 == 0) {
        int threads = ((H / 4 + 31) / 32) * 32;
        if (threads > 256) threads = 256;
        if ((int64_t)threads * 4 * RMS_MAX_ITER >= H) {
            ACORN_DISPATCH_DTYPE(dtype, T, return acorn_launch(add_rmsnorm_vec_kernel<T>, dim3(rows), dim3(threads), 0,
                                                               stream, resid32, (const T*)delta, w, (T*)out, row_idx,
                                                               H, eps));
        }
    }
    const int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
    ACORN_DISPATCH_DTYPE(dtype, T, return acorn_launch(add_rmsnorm_kernel<T>, dim3(rows), dim3(threads), 0, stream,
                                                       resid32, (const T*)delta, w, (T*)out, row_idx, H, eps));
    return ACORN_ERR_UNSUPPORTED;
}

// ---------------------------------------------------------------- SwiGLU
// out[t, i] = silu(gate) * up,   silu(z) = z / (1 + exp(-z)).  A row of gu holds, per block of b
// outputs, b gate values then b up values: gate of output i at (i / b) * 2b + i % b, up b further.
// b = I is the plain layout [gate | up].
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gu, T* __restrict__ out, int64_t total, int I, int b) {
    pdl_wait();
    pdl_trigger();
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (int64_t)gridDim.x * blockDim.x) {
        const int64_t t = idx / I;
        const int i = (int)(idx - t * I);
        const int64_t gi = t * 2 * I + (int64_t)(i / b) * 2 * b + i % b;
        const float g = to_float(gu[gi]);
        const float u = to_float(gu[gi + b]);
        out[idx] = from_float<T>(g / (1.f + expf(-g)) * u);
    }
}

// bfloat16 rows whose block width b is a multiple of 8: 16-byte loads and stores (b8 = b / 8).
// blockIdx.y is the token, so that no index is divided by the row width; a thread takes two
// 16-byte chunks of outputs a step (four loads in flight).
__global__ void swiglu_bf16x8_kernel(const bf16* __restrict__ gu, bf16* __restrict__ out, int I8, int b8) {
    pdl_wait();
    pdl_trigger();
    const bf16* row = gu + (int64_t)blockIdx.y * I8 * 16;
    bf16* orow = out + (int64_t)blockIdx.y * I8 * 8;
    auto one = [&](const uint4& g4, const uint4& u4) -> uint4 {
        const uint32_t gw[4] = {g4.x, g4.y, g4.z, g4.w}, uw[4] = {u4.x, u4.y, u4.z, u4.w};
        uint32_t ow[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float2 g = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&gw[k]));
            const float2 u = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&uw[k]));
            // exp and the quotient by the fast float32 instructions (relative error about 2^-22, far below
            // the bfloat16 rounding of the result): with the exact ones the kernel is bound by arithmetic
            __nv_bfloat162 o = __floats2bfloat162_rn(__fdividef(g.x, 1.f + __expf(-g.x)) * u.x,
                                                     __fdividef(g.y, 1.f + __expf(-g.y)) * u.y);
            ow[k] = *reinterpret_cast<uint32_t*>(&o);
        }
        return make_uint4(ow[0], ow[1], ow[2], ow[3]);
    };
    const int stride = gridDim.x * blockDim.x;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < I8; i += 2 * stride) {
        const int i2 = i + stride;
        const int gi = (i / b8) * 2 * b8 + i % b8;
        const uint4 g4 = *reinterpret_cast<const uint4*>(row + (int64_t)gi * 8);
        const uint4 u4 = *reinterpret_cast<const uint4*>(row + (int64_t)(gi + b8) * 8);
        if (i2 < I8) {
            const int gj = (i2 / b8) * 2 * b8 + i2 % b8;
            const uint4 g5 = *reinterpret_cast<const uint4*>(row + (int64_t)gj * 8);
            const uint4 u5 = *reinterpret_cast<const uint4*>(row + (int64_t)(gj + b8) * 8);
            *reinterpret_cast<uint4*>(orow + (int64_t)i2 * 8) = one(g5, u5);
        }
        *reinterpret_cast<uint4*>(orow + (int64_t)i * 8) = one(g4, u4);
    }
}

extern "C" int acorn_swiglu(const void* gu, void* out, int tokens, int I, int block, int dtype,
                            cudaStream_t stream) {
    const int64_t total = (int64_t)tokens * I;
    if (total <= 0) return 0;
    if (block <= 0 || I % block != 0) return ACORN_ERR_UNSUPPORTED;
    if (dtype == ACORN_DTYPE_BF16 && block % 8 == 0 && tokens <= 65535) {
        const int I8 = I / 8;
        int bx = (I8 + 511) / 512;                  // 256 threads, two chunks each
        if (bx < 1) bx = 1;
        return acorn_launch(swiglu_bf16x8_kernel, dim3(bx, tokens), dim3(256), 0, stream, (const bf16*)gu, (bf16*)out,
                            I8, block / 8);
    }
    int64_t blocks = (total + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    ACORN_DISPATCH_DTYPE(dtype, T, return acorn_launch(swiglu_kernel<T>, dim3((int)blocks), dim3(256), 0, stream,
                                                       (const T*)gu, (T*)out, total, I, block));
    return ACORN_ERR_UNSUPPORTED;
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
