// Shared device helpers for the sm_100a kernels: bf16 packing, 128-bit loads,
// warp/block reductions and the status codes every C-ABI entry point returns.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>

#include "../../include/iron_b200.h"

namespace iron {

constexpr int kWarp = 32;
constexpr int kSMs = 148;  // B200: 2 dies x 74 SMs; grids are sized in multiples of this

// ---- bf16 <-> f32 ---------------------------------------------------------
__device__ __forceinline__ float bf16_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }

// Round-to-nearest-even f32 -> bf16, returned as the f32 it represents.
__device__ __forceinline__ float round_bf16(float x) {
  return __bfloat162float(__float2bfloat16_rn(x));
}
// The same rounding (to nearest even) on the integer pipe, and the packing of two values that
// are bf16 already: the conversion instructions share the special-function unit with exp2 and
// the reciprocal, which an HBM-bound kernel with several roundings an element runs out of first.
__device__ __forceinline__ float round_bf16_alu(float x) {
  uint32_t u = __float_as_uint(x);
  if ((u & 0x7fffffffu) > 0x7f800000u) return x;   // NaN
  u += 0x7fffu + ((u >> 16) & 1u);
  return __uint_as_float(u & 0xffff0000u);
}
__device__ __forceinline__ uint32_t pack_bf16x2_exact(float lo, float hi) {
  return __byte_perm(__float_as_uint(lo), __float_as_uint(hi), 0x7632);
}
__device__ __forceinline__ uint16_t f2bf(float x) {
  return __bfloat16_as_ushort(__float2bfloat16_rn(x));
}
// Two floats rounded to bf16 (to nearest even) in one conversion instruction: conversions run
// on the special-function unit, so one per pair instead of one per value matters.
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
__device__ __forceinline__ void unpack8(const uint4& v, float* f) {
  f[0] = bf16_lo(v.x); f[1] = bf16_hi(v.x);
  f[2] = bf16_lo(v.y); f[3] = bf16_hi(v.y);
  f[4] = bf16_lo(v.z); f[5] = bf16_hi(v.z);
  f[6] = bf16_lo(v.w); f[7] = bf16_hi(v.w);
}
__device__ __forceinline__ uint4 pack8(const float* f) {
  uint4 v;
  v.x = pack_bf16x2(f[0], f[1]); v.y = pack_bf16x2(f[2], f[3]);
  v.z = pack_bf16x2(f[4], f[5]); v.w = pack_bf16x2(f[6], f[7]);
  return v;
}

// ---- 128-bit global loads -------------------------------------------------
// Streaming load for data read exactly once (weights): bypass L1.
__device__ __forceinline__ uint4 ld_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
// The 256-bit form sm_100 adds: one 32-byte request per lane, evict-first in L2 so a
// streamed weight matrix does not push the activations and the KV cache out of it.
// `p` must be 32-byte aligned.
__device__ __forceinline__ void ld_stream256(const void* p, uint4& lo, uint4& hi) {
  asm volatile(
      "ld.global.nc.L1::no_allocate.L2::evict_first.v8.u32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
      : "=r"(lo.x), "=r"(lo.y), "=r"(lo.z), "=r"(lo.w), "=r"(hi.x), "=r"(hi.y), "=r"(hi.z),
        "=r"(hi.w)
      : "l"(p));
}
// Plain cached load for data other CTAs re-read (activations, tables).
__device__ __forceinline__ uint4 ld_cached(const void* p) {
  return *reinterpret_cast<const uint4*>(p);
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}

// ---- reductions -----------------------------------------------------------
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
// Sum over the CTA; `scratch` holds at least 32 floats. Every thread gets the result.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarp = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();  // scratch may still be read from a previous call
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float t = (lane < nwarp) ? scratch[lane] : 0.f;
  return warp_sum(t);
}

// ---- programmatic dependent launch -----------------------------------------
// A kernel launched with the programmatic-serialization attribute may start while its
// predecessor in the stream still runs; `pdl_wait` blocks until the predecessor's
// memory is visible, `pdl_launch` lets the successor begin its own prologue.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---- L2 prefetch of memory a later kernel will stream ------------------------------
// A launch may carry a hint (iron_prefetch_hint): a region of weights the *next* kernels
// will read.  Each CTA asks the memory system to pull its slice into L2 with bulk
// prefetches; nothing waits for them.  Latency-bound kernels (attention over a short
// context, small GEMVs) leave HBM idle -- the hint fills that time, and the later
// kernel finds its weights in L2.
struct PrefetchHint {
  const char* ptr;
  long long bytes;
};
PrefetchHint take_prefetch_hint();   // host: returns and clears the pending hint
__device__ __forceinline__ void prefetch_l2_slice(const PrefetchHint& h, int cta, int ctas) {
  if (h.bytes <= 0) return;
  constexpr long long kPiece = 16384;
  long long per = (h.bytes + ctas - 1) / ctas;
  per = (per + kPiece - 1) / kPiece * kPiece;
  const long long lo = (long long)cta * per;
  const long long hi = lo + per < h.bytes ? lo + per : h.bytes;
  for (long long off = lo; off < hi; off += kPiece) {
    const unsigned int sz = (unsigned int)((hi - off < kPiece ? hi - off : kPiece) & ~15ll);
    if (sz) asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(h.ptr + off), "r"(sz) : "memory");
  }
}

// SiLU as the reference's chain computes it: f32 x*sigmoid(x), rounded once to bf16 by the
// caller.  The hardware's exp2 and reciprocal (a few float32 ulps) are far inside that rounding;
// a huge negative x gives exp = inf and the quotient 0, the limit.
__device__ __forceinline__ float silu_f32(float x) { return __fdividef(x, 1.0f + __expf(-x)); }

// Programmatic dependent launch can be switched off process-wide (iron_set_pdl): every
// launch helper asks here how many launch attributes to attach.
int pdl_attr_count();
inline void fill_pdl_attr(cudaLaunchConfig_t& cfg, cudaLaunchAttribute* attr) {
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_attr_count();
}

inline int check_launch() {
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? IRON_OK : IRON_ERR_LAUNCH;
}
inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// The current device's ordinal when it is below 64, else -1.
static inline int current_device() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return -1;
  return dev;
}

// Something done once per device (a kernel's dynamic-shared-memory limit is a per-device
// attribute): one bit per device ordinal, safe to race on from several host threads.
struct DeviceOnce {
  std::atomic<unsigned long long> bits{0};
  bool done() const {
    const int dev = current_device();
    return dev >= 0 && ((bits.load(std::memory_order_acquire) >> dev) & 1ull);
  }
  void mark() {
    const int dev = current_device();
    if (dev >= 0) bits.fetch_or(1ull << dev, std::memory_order_release);
  }
};

}  // namespace iron
