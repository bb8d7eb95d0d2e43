// Register-buffered weight streaming shared by the GEMV kernels and the decode-step kernel:
// a warp's work item is 2 KB of each of two weight rows, issued as 256-bit (or 128-bit)
// streaming loads into registers and consumed against the activation vector in shared memory.
#pragma once
#include "common.cuh"

namespace iron {

__device__ __forceinline__ float dot8(const uint4& a, const uint4& b, float acc) {
  acc = fmaf(bf16_lo(a.x), bf16_lo(b.x), acc);
  acc = fmaf(bf16_hi(a.x), bf16_hi(b.x), acc);
  acc = fmaf(bf16_lo(a.y), bf16_lo(b.y), acc);
  acc = fmaf(bf16_hi(a.y), bf16_hi(b.y), acc);
  acc = fmaf(bf16_lo(a.z), bf16_lo(b.z), acc);
  acc = fmaf(bf16_hi(a.z), bf16_hi(b.z), acc);
  acc = fmaf(bf16_lo(a.w), bf16_lo(b.w), acc);
  acc = fmaf(bf16_hi(a.w), bf16_hi(b.w), acc);
  return acc;
}

// One work item of a warp: kItem 16-byte chunks per lane of each of the pair's two rows
// (2 KB per row per warp), held in registers between issue and use.
constexpr int kItem = 4;
struct Item {
  uint4 a[kItem], b[kItem];
};

// WIDE: K % 16 == 0 and 32-byte aligned rows, so the weights move as 256-bit loads.
// Lane `lane` owns chunks (c0 + lane*2 + {0,1}) and (c0 + 64 + lane*2 + {0,1}) when WIDE,
// else chunks c0 + lane + 32*u.
template <bool WIDE>
__device__ __forceinline__ void issue(Item& it, const uint4* qa, const uint4* qb, int c0, int lane,
                                      int c_hi, bool live) {
#pragma unroll
  for (int u = 0; u < kItem; ++u) { it.a[u] = make_uint4(0, 0, 0, 0); it.b[u] = make_uint4(0, 0, 0, 0); }
  if (!live) return;
  if (WIDE) {
#pragma unroll
    for (int u = 0; u < kItem / 2; ++u) {
      const int c = c0 + 64 * u + 2 * lane;
      if (c < c_hi) {
        ld_stream256(qa + c, it.a[2 * u], it.a[2 * u + 1]);
        ld_stream256(qb + c, it.b[2 * u], it.b[2 * u + 1]);
      }
    }
  } else {
#pragma unroll
    for (int u = 0; u < kItem; ++u) {
      const int c = c0 + 32 * u + lane;
      if (c < c_hi) {
        it.a[u] = ld_stream(qa + c);
        it.b[u] = ld_stream(qb + c);
      }
    }
  }
}

template <bool WIDE>
__device__ __forceinline__ void consume(const Item& it, const uint4* xs, int c0, int lane, int c_hi,
                                        float& acc0, float& acc1) {
#pragma unroll
  for (int u = 0; u < kItem; ++u) {
    const int c = WIDE ? (c0 + 64 * (u >> 1) + 2 * lane + (u & 1)) : (c0 + 32 * u + lane);
    if (c < c_hi) {
      const uint4 xv = xs[c];
      acc0 = dot8(it.a[u], xv, acc0);
      acc1 = dot8(it.b[u], xv, acc1);
    }
  }
}

}  // namespace iron
