// Entry point of the kernel library for callers that cannot allocate device memory.
//
// It has no counterpart in the reference (ErnestW2019/acorninfer), whose kernels get all their buffers
// from PyTorch's allocator.  Some hosts of this library are not in that position: a process
// that was handed a fixed device-memory budget and must not grow it, a plug-in running inside
// another runtime's stream callback or capture set-up where cudaMalloc is forbidden or would
// synchronise the device, an embedding in a language binding that has no allocator of its own.
// Split-K decode attention normally needs scratch memory for the per-split partial results;
// this variant keeps that scratch in a fixed array inside the library instead.
//
// Limits and rules
//   * The scratch is a file-scope device array of ACORN_NOALLOC_SCRATCH_FLOATS floats (8 MiB).
//     Every GPU that loads the library holds it until the process exits.
//   * A call needs n * nq * num_splits * (d + 1) floats of it (nothing with num_splits == 1);
//     a call that needs more is refused with ACORN_ERR_SCRATCH_LIMIT and computes nothing.
//     acorn_noalloc_last_error() then says how much was asked for.
//   * The first call on a device looks up the array's device address (once per device, with
//     that device current).  Make that first call outside any stream capture.
//   * All calls share the one array and it keeps the last call's contents.  Nothing in it has
//     to start at zero: every slot a call reads was written by that call first.  Two calls
//     that overlap on the GPU (different streams, no dependency) race on it: order them.
//   * The entry point calls no cudaMalloc, cudaFree or other allocating routine.
//
// Inputs and outputs are the caller's, exactly as for acorn_attention_decode (see
// attention_decode.cu): raw device pointers, sizes, a stream; the result is the launch status.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#define ACORN_NOALLOC_SCRATCH_FLOATS (2u * 1024u * 1024u)
#define ACORN_ERR_SCRATCH_LIMIT 10002

#ifdef __cplusplus
extern "C" {
#endif

int acorn_attention_decode_noalloc(const void* q, int64_t q_stride, void* out, const void* k_pages,
                                   const void* v_pages, const int* block_table, const int* page_base,
                                   int table_stride, const int* token_row, const int* positions,
                                   const int* token_list, int n, int nq, int nkv, int d, int P, float scale,
                                   int window, int num_splits, cudaStream_t stream);

// Floats of scratch a call with these sizes needs (0 when num_splits == 1).
int64_t acorn_attention_decode_noalloc_needs(int n, int nq, int d, int num_splits);

// Text of the last refusal of this thread's calls ("" if none).
const char* acorn_noalloc_last_error(void);

#ifdef __cplusplus
}
#endif
