// The word of pinned host memory through which kernels report a bounded wait that gave up
// (see tc_fail in tcgen05_helpers.cuh), and a kernel that reports through it on request, so that
// the path from a kernel to the host's exception can be tested without a kernel going wrong.
#include "tcgen05_helpers.cuh"

__device__ int g_selftest_flag = 0;

extern "C" int acorn_error_word_alloc(int** host_ptr, int** device_ptr) {
    cudaError_t e = cudaHostAlloc(reinterpret_cast<void**>(host_ptr), 64, cudaHostAllocMapped);
    if (e != cudaSuccess) return (int)e;
    **host_ptr = 0;
    return (int)cudaHostGetDevicePointer(reinterpret_cast<void**>(device_ptr), *host_ptr, 0);
}

__global__ void error_word_selftest_kernel(int point) {
    pdl_wait();
    pdl_trigger();
    if (threadIdx.x == 0) tc_fail(&g_selftest_flag, point, ACORN_KERNEL_SELFTEST);
}

extern "C" int acorn_error_word_selftest(int point, cudaStream_t stream) {
    return acorn_launch(error_word_selftest_kernel, dim3(1), dim3(32), 0, stream, point);
}

ACORN_ERROR_WORD_SETTER(acorn_selftest_set_error_word)
