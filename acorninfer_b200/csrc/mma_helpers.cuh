// Warp-level tensor-core helpers shared by the bfloat16 attention kernels:
// mma.sync m16n8k16 (bf16 x bf16 -> f32), ldmatrix, cp.async with zero fill.
//
// Fragment layout of m16n8k16 (g = lane / 4, t = lane % 4):
//   A (16x16, row-major): a[0] = (row g,   k 2t..2t+1)   a[1] = (row g+8, k 2t..2t+1)
//                         a[2] = (row g,   k 2t+8..+9)   a[3] = (row g+8, k 2t+8..+9)
//   B (16x8,  col-major): b[0] = (k 2t..2t+1, n g)       b[1] = (k 2t+8..+9, n g)
//   C (16x8):             c[0], c[1] = (row g, col 2t, 2t+1)   c[2], c[3] = (row g+8, col 2t, 2t+1)
#pragma once

#include "common.cuh"

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t smem_addr(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}

// Four 8x8 bf16 matrices; lane l gives the address of row (l % 8) of matrix (l / 8).
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}

__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}

// 16-byte asynchronous copy global -> shared; with valid == false the destination is zero-filled
// and the source is not read.
__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src, bool valid) {
    const int bytes = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" :: "r"(dst), "l"(src), "r"(bytes));
}

__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }

template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" :: "n"(N));
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// max / sum over the four lanes that hold one row of a C fragment
__device__ __forceinline__ float quad_max(float v) {
    v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 1));
    return fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 2));
}

__device__ __forceinline__ float quad_sum(float v) {
    v += __shfl_xor_sync(0xffffffffu, v, 1);
    return v + __shfl_xor_sync(0xffffffffu, v, 2);
}

// Copies `rows` rows of D bf16 each (keys key0 .. key0+rows-1 of one kv head, looked up through
// the block table) into shared memory with row stride LDS elements.  Keys outside [lo, hi) are
// zero-filled.  `table` already points at logical page 0 of the row.  The page size is a power
// of two, 1 << logP.
template <int D, int LDS, int THREADS>
__device__ __forceinline__ void load_kv_rows(bf16* sdst, const bf16* __restrict__ pages,
                                             const int* __restrict__ table, int key0, int rows, int lo, int hi,
                                             int logP, int nkv, int kvh) {
    constexpr int SEGS = D / 8;
    const int pmask = (1 << logP) - 1;
    for (int idx = threadIdx.x; idx < rows * SEGS; idx += THREADS) {
        const int row = idx / SEGS, seg = idx - row * SEGS;
        const int key = key0 + row;
        const bool valid = key >= lo && key < hi;
        const bf16* src = pages;
        if (valid) {
            const int page = __ldg(table + (key >> logP));
            src = pages + (((((int64_t)page * nkv + kvh) << logP) + (key & pmask)) * D + seg * 8);
        }
        cp_async_16(smem_addr(sdst + row * LDS + seg * 8), src, valid);
    }
}

// The same for K and V together: a key's row has the same offset in both page tensors, so the
// block-table lookup and the address arithmetic are done once for the pair.
template <int D, int LDS, int THREADS>
__device__ __forceinline__ void load_kv_pair_rows(bf16* sk, bf16* sv, const bf16* __restrict__ k_pages,
                                                  const bf16* __restrict__ v_pages, const int* __restrict__ table,
                                                  int key0, int rows, int lo, int hi, int logP, int nkv, int kvh) {
    constexpr int SEGS = D / 8;
    const int pmask = (1 << logP) - 1;
    for (int idx = threadIdx.x; idx < rows * SEGS; idx += THREADS) {
        const int row = idx / SEGS, seg = idx - row * SEGS;
        const int key = key0 + row;
        const bool valid = key >= lo && key < hi;
        int64_t off = 0;
        if (valid) {
            const int page = __ldg(table + (key >> logP));
            off = ((((int64_t)page * nkv + kvh) << logP) + (key & pmask)) * D + seg * 8;
        }
        const int soff = row * LDS + seg * 8;
        cp_async_16(smem_addr(sk + soff), k_pages + off, valid);
        cp_async_16(smem_addr(sv + soff), v_pages + off, valid);
    }
}

// log2 of a power of two, -1 otherwise (host side).
static inline int acorn_log2_exact(int v) {
    if (v <= 0 || (v & (v - 1))) return -1;
    int l = 0;
    while ((1 << l) < v) ++l;
    return l;
}
