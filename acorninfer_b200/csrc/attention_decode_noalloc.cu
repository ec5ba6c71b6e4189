// Split-K decode attention for callers that cannot allocate: the scratch for the per-split
// partial results lives in a fixed device array of this file.  See acorn_noalloc.h for who
// needs this, the size limit and the sharing rules.  The computation is the existing
// acorn_attention_decode; only the origin of its scratch differs.
#include "acorn_noalloc.h"

#include <stdio.h>

#include "common.cuh"

// The existing entry point (attention_decode.cu); its scratch arguments are filled in here.
extern "C" int acorn_attention_decode(const void* q, int64_t q_stride, void* out, const void* k_pages,
                                      const void* v_pages, const int* block_table, const int* page_base,
                                      int table_stride, const int* token_row, const int* positions,
                                      const int* token_list, int n, int nq, int nkv, int d, int P, float scale,
                                      int window, int num_splits, float* part_o, float* part_lse,
                                      cudaStream_t stream);

// The scratch itself.  In host code this name is only a stand-in for the symbol, not a device
// address: a kernel must be given what cudaGetSymbolAddress returns for it.
static __device__ __align__(256) float g_noalloc_scratch[ACORN_NOALLOC_SCRATCH_FLOATS];

#define NOALLOC_MAX_DEVICES 64
static float* g_scratch_addr[NOALLOC_MAX_DEVICES];      // per device, filled at its first call
static thread_local char g_last_error[256] = "";

extern "C" const char* acorn_noalloc_last_error(void) { return g_last_error; }

extern "C" int64_t acorn_attention_decode_noalloc_needs(int n, int nq, int d, int num_splits) {
    if (num_splits <= 1) return 0;
    return (int64_t)n * nq * num_splits * ((int64_t)d + 1);
}

// Device address of the scratch array on the current device; looked up once per device.
static int scratch_for_current_device(float** ptr) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= NOALLOC_MAX_DEVICES) {
        snprintf(g_last_error, sizeof(g_last_error), "device index %d beyond the %d this entry point tracks", dev,
                 NOALLOC_MAX_DEVICES);
        return ACORN_ERR_UNSUPPORTED;
    }
    if (g_scratch_addr[dev] == nullptr) {
        void* addr = nullptr;
        e = cudaGetSymbolAddress(&addr, g_noalloc_scratch);
        if (e != cudaSuccess) {
            snprintf(g_last_error, sizeof(g_last_error), "cudaGetSymbolAddress failed on device %d: %s", dev,
                     cudaGetErrorString(e));
            return (int)e;
        }
        g_scratch_addr[dev] = static_cast<float*>(addr);
    }
    *ptr = g_scratch_addr[dev];
    return 0;
}

extern "C" int acorn_attention_decode_noalloc(const void* q, int64_t q_stride, void* out, const void* k_pages,
                                              const void* v_pages, const int* block_table, const int* page_base,
                                              int table_stride, const int* token_row, const int* positions,
                                              const int* token_list, int n, int nq, int nkv, int d, int P,
                                              float scale, int window, int num_splits, cudaStream_t stream) {
    g_last_error[0] = 0;
    const int64_t needs = acorn_attention_decode_noalloc_needs(n, nq, d, num_splits);
    if (needs > (int64_t)ACORN_NOALLOC_SCRATCH_FLOATS) {
        snprintf(g_last_error, sizeof(g_last_error),
                 "decode attention without allocation: %d tokens x %d heads x %d splits x (%d + 1) = %lld floats of "
                 "scratch wanted, the fixed array holds %u; use fewer splits or tokens per call",
                 n, nq, num_splits, d, (long long)needs, ACORN_NOALLOC_SCRATCH_FLOATS);
        return ACORN_ERR_SCRATCH_LIMIT;
    }
    float* part_o = nullptr;
    float* part_lse = nullptr;
    if (num_splits > 1) {
        float* base = nullptr;
        const int rc = scratch_for_current_device(&base);
        if (rc != 0) return rc;
        part_o = base;                                              // [n, nq, splits, d]
        part_lse = base + (int64_t)n * nq * num_splits * d;         // [n, nq, splits]
    }
    return acorn_attention_decode(q, q_stride, out, k_pages, v_pages, block_table, page_base, table_stride, token_row,
                                  positions, token_list, n, nq, nkv, d, P, scale, window, num_splits, part_o, part_lse,
                                  stream);
}
