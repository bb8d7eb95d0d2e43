// Row-wise softmax: y[r, :n] = softmax(v[r, :n]), zeros past n, with
//   v = x (+ addend), then cap * tanh(v / cap) when a soft cap is given,
// everything in f32 and y rounded once to bf16.  x is bf16 or f32; the addend is f32.
//
// A row is read three times (maximum, sum of exponentials, output); the second and third
// reads come from L1/L2, so a launch moves each input row from HBM once and writes each
// output row once.  Short rows (<= 1024 columns) take one warp each, eight rows per CTA;
// longer rows one CTA each.  The sum is taken in a fixed order for a given shape, so equal
// inputs give equal outputs.
#include "common.cuh"

namespace iron {

struct SoftmaxParams {
  const void* x;
  const float* addend;
  __nv_bfloat16* y;
  int rows, cols, length;
  const int* d_length;
  float cap;  // 0: none
};

template <bool F32>
__device__ __forceinline__ void load8(const SoftmaxParams& p, size_t at, float* f) {
  if constexpr (F32) {
    const float4 a = *reinterpret_cast<const float4*>(static_cast<const float*>(p.x) + at);
    const float4 b = *reinterpret_cast<const float4*>(static_cast<const float*>(p.x) + at + 4);
    f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
  } else {
    unpack8(ld_cached(static_cast<const __nv_bfloat16*>(p.x) + at), f);
  }
  if (p.addend) {
    const float4 a = *reinterpret_cast<const float4*>(p.addend + at);
    const float4 b = *reinterpret_cast<const float4*>(p.addend + at + 4);
    f[0] += a.x; f[1] += a.y; f[2] += a.z; f[3] += a.w; f[4] += b.x; f[5] += b.y; f[6] += b.z; f[7] += b.w;
  }
  if (p.cap != 0.f) {
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] = p.cap * tanhf(f[j] / p.cap);
  }
}

// GROUP threads share a row: 32 (a warp) or 256 (the CTA).
template <int GROUP, bool F32>
__global__ void __launch_bounds__(256) softmax_kernel(const SoftmaxParams p) {
  __shared__ float red[8];
  pdl_wait();
  pdl_launch();
  constexpr int kRowsPerCta = 256 / GROUP;
  const int lane = threadIdx.x % GROUP;
  const int n = p.d_length ? max(0, min(*p.d_length, p.cols)) : p.length;
  const int nch = (n + 7) >> 3, all = p.cols >> 3;
  auto group_max = [&](float v) {
#pragma unroll
    for (int off = 16; off; off >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, off));
    if constexpr (GROUP == 256) {
      __syncthreads();
      if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
      __syncthreads();
      v = red[0];
#pragma unroll
      for (int w = 1; w < 8; ++w) v = fmaxf(v, red[w]);
    }
    return v;
  };
  auto group_sum = [&](float v) {
#pragma unroll
    for (int off = 16; off; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    if constexpr (GROUP == 256) {
      __syncthreads();
      if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
      __syncthreads();
      v = red[0];
#pragma unroll
      for (int w = 1; w < 8; ++w) v += red[w];
    }
    return v;
  };
  // a CTA-wide group shares r, so its barriers are uniform; warp groups use none
  for (int r = blockIdx.x * kRowsPerCta + threadIdx.x / GROUP; r < p.rows; r += gridDim.x * kRowsPerCta) {
    const size_t base = (size_t)r * p.cols;
    float m = -INFINITY;
    for (int i = lane; i < nch; i += GROUP) {
      float f[8];
      load8<F32>(p, base + (size_t)i * 8, f);
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (i * 8 + j < n) m = fmaxf(m, f[j]);
    }
    m = group_max(m);
    float s = 0.f;
    for (int i = lane; i < nch; i += GROUP) {
      float f[8];
      load8<F32>(p, base + (size_t)i * 8, f);
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (i * 8 + j < n) s += __expf(f[j] - m);
    }
    s = group_sum(s);
    const float inv = 1.0f / s;
    uint4* yr = reinterpret_cast<uint4*>(p.y + base);
    for (int i = lane; i < all; i += GROUP) {
      float f[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      if (i < nch) {
        load8<F32>(p, base + (size_t)i * 8, f);
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] = (i * 8 + j < n) ? __expf(f[j] - m) * inv : 0.f;
      }
      yr[i] = pack8(f);
    }
  }
}

}  // namespace iron

using namespace iron;

extern "C" int iron_softmax_bf16(const void* x, int x_is_f32, const float* addend, void* y, int rows, int cols,
                                 int length, const int* d_length, float soft_cap, iron_stream_t stream) {
  if (rows <= 0 || cols <= 0 || (cols & 7) || length < 0 || length > cols) return IRON_ERR_SHAPE;
  if (!x || !y || !(soft_cap >= 0.f)) return IRON_ERR_SHAPE;
  if (!aligned16(x) || !aligned16(y) || (addend && !aligned16(addend))) return IRON_ERR_ALIGN;
  SoftmaxParams p = {x, addend, (__nv_bfloat16*)y, rows, cols, length, d_length, soft_cap};
  const bool warp_rows = cols <= 1024;
  const int ctas = warp_rows ? (rows + 7) / 8 : rows;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(ctas < kSMs * 8 ? ctas : kSMs * 8));
  cfg.blockDim = dim3(256);
  cfg.stream = (cudaStream_t)stream;
  cudaLaunchAttribute attr[1];
  fill_pdl_attr(cfg, attr);
  cudaError_t e;
  if (warp_rows)
    e = x_is_f32 ? cudaLaunchKernelEx(&cfg, softmax_kernel<32, true>, p)
                 : cudaLaunchKernelEx(&cfg, softmax_kernel<32, false>, p);
  else
    e = x_is_f32 ? cudaLaunchKernelEx(&cfg, softmax_kernel<256, true>, p)
                 : cudaLaunchKernelEx(&cfg, softmax_kernel<256, false>, p);
  return e == cudaSuccess ? IRON_OK : IRON_ERR_LAUNCH;
}
