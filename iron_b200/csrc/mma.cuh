// Warp-level tensor-core helpers (mma.sync m16n8k16, bf16 x bf16 -> f32) and the ldmatrix
// forms that feed it, for the kernels whose tiles are too small or too irregular for the
// tcgen05 path (a decode step's attention per KV group, the chunked selective scan).
//
// Fragment layouts, with g = lane / 4 and t = lane % 4:
//   A (16 x 16, row-major)   a0: (row g,     k 2t, 2t+1)    a1: (row g + 8, k 2t, 2t+1)
//                            a2: (row g,     k 2t+8, +9)    a3: (row g + 8, k 2t+8, +9)
//   B (16 x 8, "col")        b0: (k 2t, 2t+1; n g)          b1: (k 2t+8, +9; n g)
//   C / D (16 x 8, f32)      c0, c1: (row g, n 2t, 2t+1)    c2, c3: (row g + 8, n 2t, 2t+1)
#pragma once
#include "common.cuh"

namespace iron {

__device__ __forceinline__ void mma_bf16_16816(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}

// The A fragment of the 16 x 16 block at (row0, k0) of a row-major bf16 matrix in shared
// memory (`pitch` elements between rows; rows 16-byte aligned).
__device__ __forceinline__ void load_a_rowmajor(uint32_t* a, const __nv_bfloat16* base, int pitch, int row0, int k0,
                                                int lane) {
  const int r = row0 + (lane & 7) + ((lane >> 3) & 1) * 8, k = k0 + (lane >> 4) * 8;
  ldsm_x4(smem_u32(base + (size_t)r * pitch + k), a[0], a[1], a[2], a[3]);
}
// The A fragment of the block (rows m0.., k0..) of A when shared memory holds A transposed:
// element A[m][k] at base[k * pitch + m].
__device__ __forceinline__ void load_a_transposed(uint32_t* a, const __nv_bfloat16* base, int pitch, int m0, int k0,
                                                  int lane) {
  const int q = lane >> 3;
  const int k = k0 + (lane & 7) + (q >> 1) * 8, m = m0 + (q & 1) * 8;
  ldsm_x4_trans(smem_u32(base + (size_t)k * pitch + m), a[0], a[1], a[2], a[3]);
}
// B fragments of two adjacent n-tiles (n0 .. n0 + 15) at k0 when shared memory holds B as
// [n][k] (k contiguous): (b[0], b[1]) for n0 .. n0 + 7 and (b[2], b[3]) for n0 + 8 .. n0 + 15.
__device__ __forceinline__ void load_b_nk(uint32_t* b, const __nv_bfloat16* base, int pitch, int n0, int k0, int lane) {
  const int n = n0 + (lane & 7) + (lane >> 4) * 8, k = k0 + ((lane >> 3) & 1) * 8;
  ldsm_x4(smem_u32(base + (size_t)n * pitch + k), b[0], b[1], b[2], b[3]);
}
// The same two n-tiles when shared memory holds B as [k][n] (n contiguous).
__device__ __forceinline__ void load_b_kn(uint32_t* b, const __nv_bfloat16* base, int pitch, int n0, int k0, int lane) {
  const int k = k0 + (lane & 7) + ((lane >> 3) & 1) * 8, n = n0 + (lane >> 4) * 8;
  ldsm_x4_trans(smem_u32(base + (size_t)k * pitch + n), b[0], b[1], b[2], b[3]);
}

}  // namespace iron
