// Shared helpers of the sm_100a kernels: element types, conversions, reductions.
//
// Every entry point is extern "C", takes raw device pointers, sizes and a stream,
// launches on that stream and returns the cudaError_t of the launch as int
// (0 = success).  Element type is chosen by a dtype code: 0 = float32, 1 = bfloat16.
// Argument validation (sizes a kernel supports, alignment) is done by the Python
// wrappers before the call; a kernel refuses what it cannot compute with
// ACORN_ERR_UNSUPPORTED rather than computing something else.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define ACORN_DTYPE_F32 0
#define ACORN_DTYPE_BF16 1
#define ACORN_ERR_UNSUPPORTED 10001

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ float to_float(float x) { return x; }
__device__ __forceinline__ float to_float(bf16 x) { return __bfloat162float(x); }

template <typename T> __device__ __forceinline__ T from_float(float x);
template <> __device__ __forceinline__ float from_float<float>(float x) { return x; }
template <> __device__ __forceinline__ bf16 from_float<bf16>(float x) { return __float2bfloat16_rn(x); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Block-wide sum; `scratch` holds at least 32 floats of shared memory.  All threads
// of the block must call it; every thread receives the total.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float t = (lane < nwarps) ? scratch[lane] : 0.f;
    t = warp_sum(t);
    return t;
}

__device__ __forceinline__ float block_max(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float t = (lane < nwarps) ? scratch[lane] : -INFINITY;
    t = warp_max(t);
    return t;
}

// Four consecutive elements as float4 (16-byte float32 / 8-byte bfloat16 accesses).
template <typename T> struct Vec4;
template <> struct Vec4<float> {
    static __device__ __forceinline__ float4 load(const float* p) { return *reinterpret_cast<const float4*>(p); }
    static __device__ __forceinline__ void store(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
};
template <> struct Vec4<bf16> {
    static __device__ __forceinline__ float4 load(const bf16* p) {
        const uint2 raw = *reinterpret_cast<const uint2*>(p);
        const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
        const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
        return make_float4(a.x, a.y, b.x, b.y);
    }
    static __device__ __forceinline__ void store(bf16* p, float4 v) {
        __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
        uint2 raw;
        raw.x = *reinterpret_cast<uint32_t*>(&a);
        raw.y = *reinterpret_cast<uint32_t*>(&b);
        *reinterpret_cast<uint2*>(p) = raw;
    }
};

#define ACORN_DISPATCH_DTYPE(dtype, T, ...)                    \
    do {                                                       \
        if ((dtype) == ACORN_DTYPE_F32) {                      \
            typedef float T;                                   \
            __VA_ARGS__;                                       \
        } else if ((dtype) == ACORN_DTYPE_BF16) {              \
            typedef bf16 T;                                    \
            __VA_ARGS__;                                       \
        } else {                                               \
            return ACORN_ERR_UNSUPPORTED;                      \
        }                                                      \
    } while (0)

static inline int acorn_launch_status() { return (int)cudaGetLastError(); }

// Function attributes (the dynamic shared memory limit) are set per device: a launcher keeps one of
// these as a static and configures its kernel the first time it runs on each device.
struct AcornPerDevice {
    bool done[64] = {};
    static int current() {
        int dev = 0;
        return cudaGetDevice(&dev) == cudaSuccess && dev >= 0 && dev < 64 ? dev : -1;
    }
    bool seen() const {
        const int dev = current();
        return dev >= 0 && done[dev];
    }
    void mark() {
        const int dev = current();
        if (dev >= 0) done[dev] = true;
    }
};

// ---------------------------------------------------------------- programmatic dependent launch
// Every kernel of this library is launched with programmatic stream serialization: it may be
// scheduled while the kernel before it in the stream is still running, and must call
// pdl_wait() before it touches global memory that an earlier kernel wrote or still reads
// (after the wait, the earlier kernel has completed and its writes are visible).  pdl_trigger()
// lets the kernel after this one be scheduled.  Launched without the attribute both are no-ops.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

#include <cstdlib>

static inline bool acorn_pdl_enabled() {
    static int on = -1;
    if (on < 0) {
        const char* e = std::getenv("ACORN_PDL");
        on = (e != nullptr && e[0] == '0') ? 0 : 1;
    }
    return on == 1;
}

template <typename... KArgs, typename... Args>
static inline int acorn_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                               Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = acorn_pdl_enabled() ? 1 : 0;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
    return e != cudaSuccess ? (int)e : (int)cudaGetLastError();
}
