// Row-wise and element-wise bf16 kernels: RMSNorm, RoPE, the unary/binary family,
// row gather/copy and the greedy argmax.  All are HBM- or latency-bound; they use
// 128-bit coalesced accesses and compute in f32 with the roundings the reference's
// operator chain performs (each operator rounds its own output to bf16 once).
#include "common.cuh"

namespace iron {

// ---------------------------------------------------------------- RMSNorm
// One CTA per row (grid-stride over rows); the row is held in registers between the
// two passes when it fits 8 chunks per thread, else re-read (L2-resident).
__global__ void __launch_bounds__(256) rmsnorm_kernel(const __nv_bfloat16* __restrict__ x,
                                                      const __nv_bfloat16* __restrict__ w,
                                                      __nv_bfloat16* __restrict__ y, int rows,
                                                      int cols, float eps, int valid,
                                                      const int* d_valid) {
  __shared__ float red[32];
  pdl_wait();
  pdl_launch();
  if (d_valid) valid = min(*d_valid, rows);
  const int nch = cols >> 3;
  for (int r = blockIdx.x; r < valid; r += gridDim.x) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)r * cols);
    uint4* yr = reinterpret_cast<uint4*>(y + (size_t)r * cols);
    float ss = 0.f;
    for (int i = threadIdx.x; i < nch; i += blockDim.x) {
      float f[8];
      unpack8(ld_cached(xr + i), f);
#pragma unroll
      for (int j = 0; j < 8; ++j) ss = fmaf(f[j], f[j], ss);
    }
    const float tot = block_sum(ss, red);
    const float inv = 1.0f / sqrtf(tot / (float)cols + eps);
    for (int i = threadIdx.x; i < nch; i += blockDim.x) {
      float f[8];
      unpack8(ld_cached(xr + i), f);
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] = round_bf16(f[j] * inv);
      if (w) {
        float g[8];
        unpack8(ld_cached(reinterpret_cast<const uint4*>(w) + i), g);
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] = f[j] * g[j];
      }
      yr[i] = pack8(f);
    }
  }
}

// RMSNorm of x * silu(gate), the tail of a Mamba2 mixer, in one pass over HBM: the product is
// rounded to bf16 as the separate SiLU and multiply steps round it (silu first, then the
// product), held in registers across the row sum, normalised with the norm's own two
// roundings.  One CTA per row; up to kGatedChunks 16-byte chunks a thread stay in registers.
constexpr int kGatedChunks = 4;
// Two gate values -> bf16x2 of silu (f32 arithmetic, one rounding), times two packed bf16 x (the product of
// two bf16 values is exact in f32, so the bf16 multiply's single rounding is the separate steps' rounding).
__device__ __forceinline__ uint32_t gated_pair(uint32_t g, uint32_t x) {
  const __nv_bfloat162 s = __floats2bfloat162_rn(silu_f32(bf16_lo(g)), silu_f32(bf16_hi(g)));
  const __nv_bfloat162 y = __hmul2(s, *reinterpret_cast<const __nv_bfloat162*>(&x));
  return *reinterpret_cast<const uint32_t*>(&y);
}
// Two packed bf16 values scaled by `inv` in f32 and rounded, times two packed bf16 weights (w == nullptr: none).
__device__ __forceinline__ uint32_t scaled_pair(uint32_t v, float inv, const uint32_t* w) {
  __nv_bfloat162 h = __floats2bfloat162_rn(bf16_lo(v) * inv, bf16_hi(v) * inv);
  if (w) h = __hmul2(h, *reinterpret_cast<const __nv_bfloat162*>(w));
  return *reinterpret_cast<const uint32_t*>(&h);
}
__global__ void __launch_bounds__(256) rmsnorm_gated_kernel(const __nv_bfloat16* __restrict__ x,
                                                            const __nv_bfloat16* __restrict__ gate,
                                                            const __nv_bfloat16* __restrict__ w,
                                                            __nv_bfloat16* __restrict__ y, int rows, int cols,
                                                            float eps, int valid, const int* d_valid) {
  __shared__ float red[32];
  pdl_wait();
  pdl_launch();
  if (d_valid) valid = min(*d_valid, rows);
  const int nch = cols >> 3, nt = blockDim.x;
  for (int r = blockIdx.x; r < valid; r += gridDim.x) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)r * cols);
    const uint4* gr = reinterpret_cast<const uint4*>(gate + (size_t)r * cols);
    uint4* yr = reinterpret_cast<uint4*>(y + (size_t)r * cols);
    uint4 xv[kGatedChunks], gv[kGatedChunks];
#pragma unroll
    for (int u = 0; u < kGatedChunks; ++u) {
      const int i = threadIdx.x + u * nt;
      if (i < nch) { xv[u] = ld_stream(xr + i); gv[u] = ld_stream(gr + i); }
    }
    float ss = 0.f;
#pragma unroll
    for (int u = 0; u < kGatedChunks; ++u) {
      const int i = threadIdx.x + u * nt;
      if (i < nch) {
        xv[u] = make_uint4(gated_pair(gv[u].x, xv[u].x), gated_pair(gv[u].y, xv[u].y), gated_pair(gv[u].z, xv[u].z),
                           gated_pair(gv[u].w, xv[u].w));
        float f[8];
        unpack8(xv[u], f);
#pragma unroll
        for (int j = 0; j < 8; ++j) ss = fmaf(f[j], f[j], ss);
      }
    }
    const float tot = block_sum(ss, red);
    const float inv = 1.0f / sqrtf(tot / (float)cols + eps);
#pragma unroll
    for (int u = 0; u < kGatedChunks; ++u) {
      const int i = threadIdx.x + u * nt;
      if (i < nch) {
        uint4 wv = make_uint4(0u, 0u, 0u, 0u);
        if (w) wv = ld_cached(reinterpret_cast<const uint4*>(w) + i);
        yr[i] = make_uint4(scaled_pair(xv[u].x, inv, w ? &wv.x : nullptr), scaled_pair(xv[u].y, inv, w ? &wv.y : nullptr),
                           scaled_pair(xv[u].z, inv, w ? &wv.z : nullptr), scaled_pair(xv[u].w, inv, w ? &wv.w : nullptr));
      }
    }
  }
}

// ---------------------------------------------------------------- LayerNorm
// One CTA per row: mean, then the biased variance about it, then the two roundings.
__global__ void __launch_bounds__(256) layernorm_kernel(const __nv_bfloat16* __restrict__ x,
                                                        const __nv_bfloat16* __restrict__ w,
                                                        __nv_bfloat16* __restrict__ y, int rows, int cols,
                                                        float eps, int valid, const int* d_valid) {
  __shared__ float red[32];
  pdl_wait();
  pdl_launch();
  if (d_valid) valid = min(*d_valid, rows);
  const int nch = cols >> 3;
  for (int r = blockIdx.x; r < valid; r += gridDim.x) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)r * cols);
    uint4* yr = reinterpret_cast<uint4*>(y + (size_t)r * cols);
    float sum = 0.f;
    for (int i = threadIdx.x; i < nch; i += blockDim.x) {
      float f[8];
      unpack8(ld_cached(xr + i), f);
#pragma unroll
      for (int j = 0; j < 8; ++j) sum += f[j];
    }
    const float mean = block_sum(sum, red) / (float)cols;
    __syncthreads();
    float ss = 0.f;
    for (int i = threadIdx.x; i < nch; i += blockDim.x) {
      float f[8];
      unpack8(ld_cached(xr + i), f);
#pragma unroll
      for (int j = 0; j < 8; ++j) { const float d = f[j] - mean; ss = fmaf(d, d, ss); }
    }
    const float inv = 1.0f / sqrtf(block_sum(ss, red) / (float)cols + eps);
    __syncthreads();
    for (int i = threadIdx.x; i < nch; i += blockDim.x) {
      float f[8];
      unpack8(ld_cached(xr + i), f);
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] = round_bf16((f[j] - mean) * inv);
      if (w) {
        float g[8];
        unpack8(ld_cached(reinterpret_cast<const uint4*>(w) + i), g);
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] = f[j] * g[j];
      }
      yr[i] = pack8(f);
    }
  }
}

// ---------------------------------------------------------------- clamp
__global__ void __launch_bounds__(256) clamp_kernel(const __nv_bfloat16* __restrict__ a, __nv_bfloat16* __restrict__ y,
                                                    long long n, float low, float high) {
  pdl_wait();
  pdl_launch();
  const long long nvec = n >> 3;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec; i += stride) {
    float f[8];
    unpack8(ld_cached(reinterpret_cast<const uint4*>(a) + i), f);
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] = fminf(fmaxf(f[j], low), high);
    reinterpret_cast<uint4*>(y)[i] = pack8(f);
  }
  for (long long i = (nvec << 3) + blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += stride)
    y[i] = __float2bfloat16_rn(fminf(fmaxf(__bfloat162float(a[i]), low), high));
}

// ---------------------------------------------------------------- RoPE
// One thread per 8 output pairs.  two_halves: pair (i, i + cols/2); else (2i, 2i+1).
__global__ void __launch_bounds__(256) rope_kernel(const __nv_bfloat16* __restrict__ x,
                                                   const __nv_bfloat16* __restrict__ angles,
                                                   __nv_bfloat16* __restrict__ y, int rows, int cols,
                                                   int rows_per_angle, int two_halves,
                                                   int angle_offset, const int* d_angle_offset,
                                                   int valid, const int* d_valid) {
  pdl_wait();
  pdl_launch();
  if (d_valid) valid = min(*d_valid, rows);
  if (d_angle_offset) angle_offset = *d_angle_offset;
  const int half = cols >> 1;
  const int per_row = half >> 3;  // groups of 8 pairs per row
  const long long total = (long long)valid * per_row;
  for (long long t = blockIdx.x * (long long)blockDim.x + threadIdx.x; t < total;
       t += (long long)gridDim.x * blockDim.x) {
    const int r = (int)(t / per_row), g = (int)(t - (long long)r * per_row);
    const int i0 = g * 8;  // first pair index
    const __nv_bfloat16* xr = x + (size_t)r * cols;
    const __nv_bfloat16* ar = angles + (size_t)(angle_offset + r / rows_per_angle) * cols;
    __nv_bfloat16* yr = y + (size_t)r * cols;
    float cs[16];  // cos,sin interleaved for pairs i0..i0+7 = columns 2*i0 .. 2*i0+15
    unpack8(ld_cached(ar + 2 * i0), cs);
    unpack8(ld_cached(ar + 2 * i0 + 8), cs + 8);
    float a[8], b[8], oa[8], ob[8];
    if (two_halves) {
      unpack8(ld_cached(xr + i0), a);
      unpack8(ld_cached(xr + half + i0), b);
    } else {
      float v[16];
      unpack8(ld_cached(xr + 2 * i0), v);
      unpack8(ld_cached(xr + 2 * i0 + 8), v + 8);
#pragma unroll
      for (int j = 0; j < 8; ++j) { a[j] = v[2 * j]; b[j] = v[2 * j + 1]; }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float c = cs[2 * j], s = cs[2 * j + 1];
      oa[j] = __fsub_rn(__fmul_rn(a[j], c), __fmul_rn(b[j], s));
      ob[j] = __fadd_rn(__fmul_rn(b[j], c), __fmul_rn(a[j], s));
    }
    if (two_halves) {
      *reinterpret_cast<uint4*>(yr + i0) = pack8(oa);
      *reinterpret_cast<uint4*>(yr + half + i0) = pack8(ob);
    } else {
      float v[16];
#pragma unroll
      for (int j = 0; j < 8; ++j) { v[2 * j] = oa[j]; v[2 * j + 1] = ob[j]; }
      *reinterpret_cast<uint4*>(yr + 2 * i0) = pack8(v);
      *reinterpret_cast<uint4*>(yr + 2 * i0 + 8) = pack8(v + 8);
    }
  }
}

// ---------------------------------------------------------------- prompt-chunk RoPE + KV write
// qkv is (rows, (H + 2G) * D) with row pitch `pitch`: q heads, then k heads, then v heads.
// q is rotated in place, k is rotated into k_cache[start + row], v copied into
// v_cache[start + row].  One thread per 8 rotation pairs (or 16 copied elements).
__global__ void __launch_bounds__(256) rope_kv_kernel(__nv_bfloat16* __restrict__ qkv, long long pitch,
                                                      const __nv_bfloat16* __restrict__ angles,
                                                      __nv_bfloat16* __restrict__ k_cache,
                                                      __nv_bfloat16* __restrict__ v_cache, int rows,
                                                      const int* d_rows, int H, int G, int D, int start,
                                                      const int* d_start, int angle_start,
                                                      const int* d_angle_start) {
  pdl_wait();
  pdl_launch();
  if (d_rows) rows = min(*d_rows, rows);
  if (d_start) start = *d_start;
  if (d_angle_start) angle_start = *d_angle_start;
  const int half = D >> 1, per_head = half >> 3, heads = H + 2 * G;
  const long long total = (long long)rows * heads * per_head;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int pg = (int)(idx % per_head);
    const int hh = (int)((idx / per_head) % heads);
    const int r = (int)(idx / ((long long)per_head * heads));
    const int i0 = pg * 8;
    __nv_bfloat16* src = qkv + (long long)r * pitch + (long long)hh * D;
    float a[8], b[8];
    unpack8(ld_cached(src + i0), a);
    unpack8(ld_cached(src + half + i0), b);
    if (hh < H + G) {
      const __nv_bfloat16* ar = angles + (size_t)(angle_start + r) * D;
      float cs[16];
      unpack8(ld_cached(ar + 2 * i0), cs);
      unpack8(ld_cached(ar + 2 * i0 + 8), cs + 8);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float c = cs[2 * j], s = cs[2 * j + 1];
        const float ya = __fsub_rn(__fmul_rn(a[j], c), __fmul_rn(b[j], s));
        const float yb = __fadd_rn(__fmul_rn(b[j], c), __fmul_rn(a[j], s));
        a[j] = ya; b[j] = yb;
      }
    }
    __nv_bfloat16* dst;
    if (hh < H) dst = src;
    else if (hh < H + G) dst = k_cache + ((size_t)(start + r) * G + (hh - H)) * D;
    else dst = v_cache + ((size_t)(start + r) * G + (hh - H - G)) * D;
    *reinterpret_cast<uint4*>(dst + i0) = pack8(a);
    *reinterpret_cast<uint4*>(dst + half + i0) = pack8(b);
  }
}

// ---------------------------------------------------------------- element-wise
__device__ __forceinline__ float ew_apply(int op, float a, float b, float s) {
  switch (op) {
    case IRON_EW_SILU: return silu_f32(a);
    case IRON_EW_ADD:
    case IRON_EW_ROW_ADD: return __fadd_rn(a, b);
    case IRON_EW_MUL:
    case IRON_EW_ROW_MUL: return __fmul_rn(a, b);
    case IRON_EW_AXPY: return __fadd_rn(__fmul_rn(s, a), b);
    case IRON_EW_SILU_MUL: return __fmul_rn(round_bf16(silu_f32(a)), b);
    case IRON_EW_SIGMOID: return 1.0f / (1.0f + expf(-a));
    case IRON_EW_GELU_SIG: return __fmul_rn(a, round_bf16(1.0f / (1.0f + expf(-__fmul_rn(1.702f, a)))));
    case IRON_EW_RELU: return fmaxf(a, 0.f);
    case IRON_EW_TANH: return tanhf(a);
    case IRON_EW_GELU_TANH: return 0.5f * a * (1.0f + tanhf(0.7978845608028654f * (a + 0.044715f * a * a * a)));
    case IRON_EW_GELU_ERF: return 0.5f * a * (1.0f + erff(a * 0.7071067811865476f));
  }
  return 0.f;
}

template <int OP>
__global__ void __launch_bounds__(256) ew_kernel(const __nv_bfloat16* __restrict__ a,
                                                 const __nv_bfloat16* __restrict__ b,
                                                 __nv_bfloat16* __restrict__ y, long long n,
                                                 int cols, float scalar) {
  pdl_wait();
  pdl_launch();
  constexpr bool kBinary = OP == IRON_EW_ADD || OP == IRON_EW_MUL || OP == IRON_EW_AXPY ||
                           OP == IRON_EW_SILU_MUL;
  constexpr bool kRow = OP == IRON_EW_ROW_ADD || OP == IRON_EW_ROW_MUL;
  const long long nvec = n >> 3;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec; i += stride) {
    float fa[8], fb[8];
    unpack8(ld_cached(reinterpret_cast<const uint4*>(a) + i), fa);
    if (kBinary) unpack8(ld_cached(reinterpret_cast<const uint4*>(b) + i), fb);
    if (kRow) {
      // cols % 8 == 0 is checked on the host, so a chunk never straddles two rows
      const long long c = (i * 8) % cols;
      unpack8(ld_cached(b + c), fb);
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) fa[j] = ew_apply(OP, fa[j], (kBinary || kRow) ? fb[j] : 0.f, scalar);
    reinterpret_cast<uint4*>(y)[i] = pack8(fa);
  }
  // ragged tail (n % 8 elements), scalar
  const long long tail0 = nvec << 3;
  for (long long i = tail0 + blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += stride) {
    const float fa = __bfloat162float(a[i]);
    float fb = 0.f;
    if (kBinary) fb = __bfloat162float(b[i]);
    if (kRow) fb = __bfloat162float(b[i % cols]);
    y[i] = __float2bfloat16_rn(ew_apply(OP, fa, fb, scalar));
  }
}

// ---------------------------------------------------------------- copy / gather
// One warp per row-chunk: rows of `row_bytes` (multiple of 16) moved as uint4.
__global__ void __launch_bounds__(256) copy_rows_kernel(const char* __restrict__ src,
                                                        char* __restrict__ dst,
                                                        const int* __restrict__ ids, int nrows,
                                                        const int* d_nrows, long long row_bytes,
                                                        long long src_pitch, long long dst_pitch,
                                                        int src_rows, int src_row0,
                                                        const int* d_src_row0, int dst_row0,
                                                        const int* d_dst_row0) {
  pdl_wait();
  pdl_launch();
  if (d_nrows) nrows = min(*d_nrows, nrows);
  if (d_src_row0) src_row0 = *d_src_row0;
  if (d_dst_row0) dst_row0 = *d_dst_row0;
  const long long vec_per_row = row_bytes >> 4;
  const long long total = (long long)nrows * vec_per_row;
  for (long long t = blockIdx.x * (long long)blockDim.x + threadIdx.x; t < total;
       t += (long long)gridDim.x * blockDim.x) {
    const long long r = t / vec_per_row, v = t - r * vec_per_row;
    long long sr;
    if (ids) {
      int id = ids[r];
      id = id < 0 ? 0 : (id >= src_rows ? src_rows - 1 : id);
      sr = id;
    } else {
      sr = src_row0 + r;
    }
    const uint4 val = *reinterpret_cast<const uint4*>(src + sr * src_pitch + v * 16);
    *reinterpret_cast<uint4*>(dst + (dst_row0 + r) * dst_pitch + v * 16) = val;
  }
}

// ---------------------------------------------------------------- argmax
// Keys order by (value, lower index first): the f32 bits made monotone, then the
// complement of the index, so a 64-bit max is numpy's first-occurrence argmax.
__device__ __forceinline__ unsigned long long argmax_key(float v, int idx) {
  uint32_t u = __float_as_uint(v);
  u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
  if (v != v) u = 0;  // NaN never wins over a number
  return ((unsigned long long)u << 32) | (uint32_t)(~(uint32_t)idx);
}
__device__ __forceinline__ unsigned long long umax64(unsigned long long a, unsigned long long b) {
  return a > b ? a : b;
}

constexpr int kArgmaxBlocks = kSMs * 2;

// workspace layout: [0] u32 arrival counter, [8 ..] u64 partial keys per block
__global__ void __launch_bounds__(256) argmax_kernel(const __nv_bfloat16* __restrict__ logits, int n,
                                                     int* token_out, const int* d_out_index,
                                                     int out_rows, int* carry_token, int* carry_position,
                                                     unsigned long long* workspace, int index_offset,
                                                     unsigned long long* key_out) {
  __shared__ unsigned long long sred[8];
  __shared__ bool last;
  pdl_wait();
  pdl_launch();
  unsigned int* counter = reinterpret_cast<unsigned int*>(workspace);
  unsigned long long* partial = workspace + 1;
  unsigned long long best = 0;
  const int nvec = n >> 3;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += gridDim.x * blockDim.x) {
    float f[8];
    unpack8(ld_cached(reinterpret_cast<const uint4*>(logits) + i), f);
#pragma unroll
    for (int j = 0; j < 8; ++j) best = umax64(best, argmax_key(f[j], index_offset + i * 8 + j));
  }
  for (int i = (nvec << 3) + blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x)
    best = umax64(best, argmax_key(__bfloat162float(logits[i]), index_offset + i));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) best = umax64(best, __shfl_xor_sync(0xffffffffu, best, o));
  if ((threadIdx.x & 31) == 0) sred[threadIdx.x >> 5] = best;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < 8; ++w) best = umax64(best, sred[w]);
    partial[blockIdx.x] = best;
    __threadfence();
    const unsigned int arrived = atomicAdd(counter, 1u);
    last = (arrived == gridDim.x - 1);
  }
  __syncthreads();
  if (last) {  // the last CTA to arrive folds the partials; nobody waits on anybody
    __threadfence();
    unsigned long long b = 0;
    for (int i = threadIdx.x; i < (int)gridDim.x; i += blockDim.x)
      b = umax64(b, *reinterpret_cast<volatile unsigned long long*>(partial + i));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) b = umax64(b, __shfl_xor_sync(0xffffffffu, b, o));
    if ((threadIdx.x & 31) == 0) sred[threadIdx.x >> 5] = b;
    __syncthreads();
    if (threadIdx.x == 0) {
      for (int w = 1; w < 8; ++w) b = umax64(b, sred[w]);
      if (key_out) {   // a shard's candidate: the draw is made from every shard's key
        *key_out = b;
        *counter = 0;
        return;
      }
      const int tok = (int)(~(uint32_t)(b & 0xffffffffull));
      // out_rows > 0 bounds the row written; when the row written IS the carried position
      // (a decoder's loop: d_out_index and carry_position are one word) the position stops
      // growing at out_rows, so a replay past the end of the caches stays inside them
      const int at = d_out_index ? *d_out_index : 0;
      if (out_rows <= 0 || (at >= 0 && at < out_rows)) token_out[at] = tok;
      if (carry_token) *carry_token = tok;
      const bool tied = out_rows > 0 && d_out_index == carry_position;
      if (carry_position && (!tied || *carry_position < out_rows)) *carry_position += 1;
      *counter = 0;  // leave the workspace ready for the next launch
    }
  }
}

template <typename... Args>
static int launch_pdl(void (*kernel)(Args...), dim3 grid, dim3 block, cudaStream_t stream,
                      Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = 0;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  fill_pdl_attr(cfg, attr);
  return cudaLaunchKernelEx(&cfg, kernel, args...) == cudaSuccess ? IRON_OK : IRON_ERR_LAUNCH;
}

static int grid_for(long long work_items, int threads) {
  long long blocks = (work_items + threads - 1) / threads;
  if (blocks < 1) blocks = 1;
  const long long cap = (long long)kSMs * 8;
  return (int)(blocks > cap ? cap : blocks);
}

}  // namespace iron

using namespace iron;

static thread_local iron::PrefetchHint g_hint = {nullptr, 0};
namespace iron {
PrefetchHint take_prefetch_hint() {
  PrefetchHint h = g_hint;
  g_hint = PrefetchHint{nullptr, 0};
  return h;
}
}  // namespace iron
extern "C" int iron_prefetch_hint(const void* ptr, long long bytes) {
  if (bytes < 0 || (bytes > 0 && !ptr) || (reinterpret_cast<uintptr_t>(ptr) & 15)) return IRON_ERR_ALIGN;
  g_hint = iron::PrefetchHint{static_cast<const char*>(ptr), bytes};
  return IRON_OK;
}
static int g_pdl_enabled = 1;
namespace iron { int pdl_attr_count() { return g_pdl_enabled ? 1 : 0; } }
extern "C" void iron_set_pdl(int enabled) { g_pdl_enabled = enabled ? 1 : 0; }
extern "C" int iron_version(void) { return 100; }
extern "C" const char* iron_arch(void) { return "sm_100a"; }

extern "C" int iron_rmsnorm_bf16(const void* x, const void* weight, void* y, int rows, int cols,
                                 float eps, int valid_rows, const int* d_valid_rows,
                                 iron_stream_t stream) {
  if (rows <= 0 || cols <= 0 || (cols & 7)) return IRON_ERR_SHAPE;
  if (valid_rows < 0 || valid_rows > rows) return IRON_ERR_SHAPE;
  if (!aligned16(x) || !aligned16(y) || (weight && !aligned16(weight))) return IRON_ERR_ALIGN;
  if (valid_rows == 0 && !d_valid_rows) return IRON_OK;
  const int upper = d_valid_rows ? rows : valid_rows;
  const int grid = upper < kSMs * 8 ? upper : kSMs * 8;
  return launch_pdl(rmsnorm_kernel, dim3(grid), dim3(256), (cudaStream_t)stream,
                    (const __nv_bfloat16*)x, (const __nv_bfloat16*)weight, (__nv_bfloat16*)y, rows,
                    cols, eps, valid_rows, d_valid_rows);
}

extern "C" int iron_rmsnorm_gated_bf16(const void* x, const void* gate, const void* weight, void* y, int rows,
                                       int cols, float eps, int valid_rows, const int* d_valid_rows,
                                       iron_stream_t stream) {
  if (rows <= 0 || cols <= 0 || (cols & 7) || cols > 256 * 8 * kGatedChunks) return IRON_ERR_SHAPE;
  if (valid_rows < 0 || valid_rows > rows) return IRON_ERR_SHAPE;
  if (!x || !gate || !y) return IRON_ERR_SHAPE;
  if (!aligned16(x) || !aligned16(gate) || !aligned16(y) || (weight && !aligned16(weight))) return IRON_ERR_ALIGN;
  if (valid_rows == 0 && !d_valid_rows) return IRON_OK;
  const int upper = d_valid_rows ? rows : valid_rows;
  // 128 threads when they cover the row with up to four chunks each (a 3072-wide row is three chunks a thread)
  const int threads = (cols >> 3) <= 128 * kGatedChunks ? 128 : 256;
  const int full = kSMs * (2048 / threads);
  const int grid = upper < full ? upper : full;
  return launch_pdl(rmsnorm_gated_kernel, dim3(grid), dim3(threads), (cudaStream_t)stream,
                    (const __nv_bfloat16*)x, (const __nv_bfloat16*)gate, (const __nv_bfloat16*)weight,
                    (__nv_bfloat16*)y, rows, cols, eps, valid_rows, d_valid_rows);
}

extern "C" int iron_layernorm_bf16(const void* x, const void* weight, void* y, int rows, int cols, float eps,
                                   int valid_rows, const int* d_valid_rows, iron_stream_t stream) {
  if (rows <= 0 || cols <= 0 || (cols & 7)) return IRON_ERR_SHAPE;
  if (valid_rows < 0 || valid_rows > rows) return IRON_ERR_SHAPE;
  if (!aligned16(x) || !aligned16(y) || (weight && !aligned16(weight))) return IRON_ERR_ALIGN;
  if (valid_rows == 0 && !d_valid_rows) return IRON_OK;
  const int upper = d_valid_rows ? rows : valid_rows;
  const int grid = upper < kSMs * 8 ? upper : kSMs * 8;
  return launch_pdl(layernorm_kernel, dim3(grid), dim3(256), (cudaStream_t)stream, (const __nv_bfloat16*)x,
                    (const __nv_bfloat16*)weight, (__nv_bfloat16*)y, rows, cols, eps, valid_rows, d_valid_rows);
}

extern "C" int iron_clamp_bf16(const void* x, void* y, long long n, float low, float high, iron_stream_t stream) {
  if (n < 0 || !(low <= high)) return IRON_ERR_SHAPE;
  if (n == 0) return IRON_OK;
  if (!aligned16(x) || !aligned16(y)) return IRON_ERR_ALIGN;
  // the bounds as bf16 values, as the reference passes them to its kernel
  const float lo = __bfloat162float(__float2bfloat16_rn(low)), hi = __bfloat162float(__float2bfloat16_rn(high));
  return launch_pdl(clamp_kernel, dim3(grid_for((n + 7) / 8, 256)), dim3(256), (cudaStream_t)stream,
                    (const __nv_bfloat16*)x, (__nv_bfloat16*)y, n, lo, hi);
}

extern "C" int iron_rope_bf16(const void* x, const void* angles, void* y, int rows, int cols,
                              int angle_rows, int two_halves, int angle_offset,
                              const int* d_angle_offset, int valid_rows, const int* d_valid_rows,
                              iron_stream_t stream) {
  if (rows <= 0 || cols < 16 || (cols & 15)) return IRON_ERR_SHAPE;
  if (angle_rows <= 0 || angle_rows > rows || rows % angle_rows) return IRON_ERR_SHAPE;
  if (valid_rows < 0 || valid_rows > rows) return IRON_ERR_SHAPE;
  if (!aligned16(x) || !aligned16(y) || !aligned16(angles)) return IRON_ERR_ALIGN;
  if (valid_rows == 0 && !d_valid_rows) return IRON_OK;
  const int upper = d_valid_rows ? rows : valid_rows;
  const long long items = (long long)upper * (cols / 16);
  return launch_pdl(rope_kernel, dim3(grid_for(items, 256)), dim3(256), (cudaStream_t)stream,
                    (const __nv_bfloat16*)x, (const __nv_bfloat16*)angles, (__nv_bfloat16*)y, rows,
                    cols, rows / angle_rows, two_halves, angle_offset, d_angle_offset, valid_rows,
                    d_valid_rows);
}

extern "C" int iron_elementwise_bf16(int op, const void* a, const void* b, void* y, long long n,
                                     int cols, float scalar, iron_stream_t stream) {
  if (n < 0) return IRON_ERR_SHAPE;
  if (n == 0) return IRON_OK;
  if (!aligned16(a) || !aligned16(y) || (b && !aligned16(b))) return IRON_ERR_ALIGN;
  const bool row = op == IRON_EW_ROW_ADD || op == IRON_EW_ROW_MUL;
  const bool binary = op == IRON_EW_ADD || op == IRON_EW_MUL || op == IRON_EW_AXPY ||
                      op == IRON_EW_SILU_MUL;
  if ((row || binary) && !b) return IRON_ERR_SHAPE;
  if (row && (cols <= 0 || (cols & 7) || n % cols)) return IRON_ERR_SHAPE;
  const dim3 grid(grid_for((n + 7) / 8, 256)), block(256);
  cudaStream_t s = (cudaStream_t)stream;
  const __nv_bfloat16 *pa = (const __nv_bfloat16*)a, *pb = (const __nv_bfloat16*)b;
  __nv_bfloat16* py = (__nv_bfloat16*)y;
#define IRON_EW_CASE(OP) \
  case OP: return launch_pdl(ew_kernel<OP>, grid, block, s, pa, pb, py, n, cols, scalar);
  switch (op) {
    IRON_EW_CASE(IRON_EW_SILU)
    IRON_EW_CASE(IRON_EW_ADD)
    IRON_EW_CASE(IRON_EW_MUL)
    IRON_EW_CASE(IRON_EW_AXPY)
    IRON_EW_CASE(IRON_EW_SILU_MUL)
    IRON_EW_CASE(IRON_EW_ROW_ADD)
    IRON_EW_CASE(IRON_EW_ROW_MUL)
    IRON_EW_CASE(IRON_EW_SIGMOID)
    IRON_EW_CASE(IRON_EW_GELU_SIG)
    IRON_EW_CASE(IRON_EW_RELU)
    IRON_EW_CASE(IRON_EW_TANH)
    IRON_EW_CASE(IRON_EW_GELU_TANH)
    IRON_EW_CASE(IRON_EW_GELU_ERF)
  }
#undef IRON_EW_CASE
  return IRON_ERR_UNSUPPORTED;
}

extern "C" int iron_copy_rows(const void* src, void* dst, const int* ids, int nrows,
                              const int* d_nrows, long long row_bytes, long long src_pitch,
                              long long dst_pitch, int src_rows, int src_row0,
                              const int* d_src_row0, int dst_row0, const int* d_dst_row0,
                              iron_stream_t stream) {
  if (nrows < 0 || row_bytes <= 0 || (row_bytes & 15) || (src_pitch & 15) || (dst_pitch & 15))
    return IRON_ERR_SHAPE;
  if (!aligned16(src) || !aligned16(dst)) return IRON_ERR_ALIGN;
  if (ids && src_rows <= 0) return IRON_ERR_SHAPE;
  if (nrows == 0) return IRON_OK;
  const long long items = (long long)nrows * (row_bytes >> 4);
  return launch_pdl(copy_rows_kernel, dim3(grid_for(items, 256)), dim3(256), (cudaStream_t)stream,
                    (const char*)src, (char*)dst, ids, nrows, d_nrows, row_bytes, src_pitch,
                    dst_pitch, src_rows, src_row0, d_src_row0, dst_row0, d_dst_row0);
}

extern "C" size_t iron_argmax_workspace_bytes(int n) {
  (void)n;
  return sizeof(unsigned long long) * (1 + kArgmaxBlocks);
}

extern "C" int iron_argmax_bf16(const void* logits, int n, int* token_out,
                                const int* d_out_index, int out_rows, int* carry_token,
                                int* carry_position, void* workspace, iron_stream_t stream) {
  if (n <= 0 || !token_out || !workspace) return IRON_ERR_SHAPE;
  if (!aligned16(logits) || (reinterpret_cast<uintptr_t>(workspace) & 7)) return IRON_ERR_ALIGN;
  int grid = (n / 8 + 255) / 256;
  grid = grid < 1 ? 1 : (grid > kArgmaxBlocks ? kArgmaxBlocks : grid);
  return launch_pdl(argmax_kernel, dim3(grid), dim3(256), (cudaStream_t)stream,
                    (const __nv_bfloat16*)logits, n, token_out, d_out_index, out_rows, carry_token,
                    carry_position, (unsigned long long*)workspace, 0, (unsigned long long*)nullptr);
}

// The greedy draw over a vocabulary split across ranks: every rank reduces its rows of the
// logits to one 64-bit key (value, then lowest global index), the keys are gathered, and the
// largest key names the token -- the same first-maximum rule as over the whole row.
__global__ void argmax_pick_kernel(const unsigned long long* __restrict__ keys, int count, int* token_out,
                                   const int* d_out_index, int out_rows, int* carry_token, int* carry_position) {
  pdl_wait();
  pdl_launch();
  if (threadIdx.x != 0) return;
  unsigned long long b = 0;
  for (int i = 0; i < count; ++i) b = umax64(b, keys[i]);
  const int tok = (int)(~(uint32_t)(b & 0xffffffffull));
  const int at = d_out_index ? *d_out_index : 0;
  if (out_rows <= 0 || (at >= 0 && at < out_rows)) token_out[at] = tok;
  if (carry_token) *carry_token = tok;
  const bool tied = out_rows > 0 && d_out_index == carry_position;
  if (carry_position && (!tied || *carry_position < out_rows)) *carry_position += 1;
}

extern "C" int iron_argmax_key_bf16(const void* logits, int n, int index_offset, void* key_out, void* workspace,
                                    iron_stream_t stream) {
  if (n <= 0 || index_offset < 0 || !key_out || !workspace) return IRON_ERR_SHAPE;
  if (!aligned16(logits) || (reinterpret_cast<uintptr_t>(workspace) & 7) || (reinterpret_cast<uintptr_t>(key_out) & 7))
    return IRON_ERR_ALIGN;
  int grid = (n / 8 + 255) / 256;
  grid = grid < 1 ? 1 : (grid > kArgmaxBlocks ? kArgmaxBlocks : grid);
  return launch_pdl(argmax_kernel, dim3(grid), dim3(256), (cudaStream_t)stream, (const __nv_bfloat16*)logits, n,
                    (int*)nullptr, (const int*)nullptr, 0, (int*)nullptr, (int*)nullptr,
                    (unsigned long long*)workspace, index_offset, (unsigned long long*)key_out);
}

extern "C" int iron_argmax_pick(const void* keys, int count, int* token_out, const int* d_out_index, int out_rows,
                                int* carry_token, int* carry_position, iron_stream_t stream) {
  if (count <= 0 || !keys || !token_out) return IRON_ERR_SHAPE;
  if (reinterpret_cast<uintptr_t>(keys) & 7) return IRON_ERR_ALIGN;
  return launch_pdl(argmax_pick_kernel, dim3(1), dim3(32), (cudaStream_t)stream, (const unsigned long long*)keys,
                    count, token_out, d_out_index, out_rows, carry_token, carry_position);
}

extern "C" int iron_rope_kv_write_bf16(void* qkv, long long pitch, const void* angles, void* k_cache,
                                       void* v_cache, int rows, const int* d_rows, int H, int G, int D,
                                       int start, const int* d_start, int angle_start,
                                       const int* d_angle_start, iron_stream_t stream) {
  if (rows < 0 || H <= 0 || G <= 0 || D < 16 || (D & 15)) return IRON_ERR_SHAPE;
  if (pitch < (long long)(H + 2 * G) * D || (pitch & 7)) return IRON_ERR_SHAPE;
  if (start < 0 || angle_start < 0) return IRON_ERR_SHAPE;
  if (!aligned16(qkv) || !aligned16(angles) || !aligned16(k_cache) || !aligned16(v_cache)) return IRON_ERR_ALIGN;
  if (rows == 0) return IRON_OK;
  const long long items = (long long)rows * (H + 2 * G) * (D / 16);
  return launch_pdl(rope_kv_kernel, dim3(grid_for(items, 256)), dim3(256), (cudaStream_t)stream,
                    (__nv_bfloat16*)qkv, pitch, (const __nv_bfloat16*)angles, (__nv_bfloat16*)k_cache,
                    (__nv_bfloat16*)v_cache, rows, d_rows, H, G, D, start, d_start, angle_start,
                    d_angle_start);
}

// ---------------------------------------------------------------- greedy draw without a workspace
// Some callers cannot hand the library scratch memory: code that runs where cudaMalloc is not
// available to it -- a host thread that must not touch the allocator (it would take the
// allocator's lock or synchronise the device), a plugin bound into a runtime that owns all
// device memory and exposes no allocation hook, or a caller already inside a region where
// allocation is illegal.  For them the argmax's cross-block scratch (one arrival counter and
// one 64-bit partial per block) lives in this file-scope device array instead.  Every GPU that
// loads the library holds these few kilobytes until the process exits.
static __device__ __align__(256) unsigned long long g_argmax_scratch[1 + iron::kArgmaxBlocks];

namespace {
constexpr int kNoAllocMaxN = 1 << 22;  // logits per call this entry point accepts
constexpr int kMaxDevices = 64;
std::atomic<unsigned long long*> g_scratch_ptr[kMaxDevices] = {};  // device address of the array, per device
}  // namespace

extern "C" int iron_argmax_noalloc_max_n(void) { return kNoAllocMaxN; }

extern "C" int iron_argmax_bf16_noalloc(const void* logits, int n, int* token_out, const int* d_out_index,
                                        int* carry_token, int* carry_position, iron_stream_t stream) {
  if (n <= 0 || !token_out) return IRON_ERR_SHAPE;
  if (n > kNoAllocMaxN) return IRON_ERR_WORKSPACE;  // more logits than the built-in scratch is stated for
  if (!aligned16(logits)) return IRON_ERR_ALIGN;
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return IRON_ERR_LAUNCH;
  if (!g_scratch_ptr[dev].load(std::memory_order_acquire)) {
    // In host code `g_argmax_scratch` is only a stand-in for the symbol: its device address
    // has to be asked for, once per device, with that device current.
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_argmax_scratch) != cudaSuccess || !p) return IRON_ERR_LAUNCH;
    g_scratch_ptr[dev].store(static_cast<unsigned long long*>(p), std::memory_order_release);
  }
  unsigned long long* scratch = g_scratch_ptr[dev].load(std::memory_order_acquire);
  cudaStream_t s = (cudaStream_t)stream;
  // The array keeps whatever the last call left: the arrival counter must start at zero.
  if (cudaMemsetAsync(scratch, 0, sizeof(unsigned long long), s) != cudaSuccess) return IRON_ERR_LAUNCH;
  int grid = (n / 8 + 255) / 256;
  grid = grid < 1 ? 1 : (grid > kArgmaxBlocks ? kArgmaxBlocks : grid);
  return launch_pdl(argmax_kernel, dim3(grid), dim3(256), s, (const __nv_bfloat16*)logits, n, token_out,
                    d_out_index, 0, carry_token, carry_position, scratch, 0, (unsigned long long*)nullptr);
}
