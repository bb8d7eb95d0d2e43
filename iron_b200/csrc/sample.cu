// The token drawn from a row of logits: temperature, then top-k, then a draw from the softmax,
// by the rule iron_b200/lm/generation.py states (and its host Sampler follows), operation for
// operation, so that host and device pick the same token from the same logits and uniform:
//   1. candidates: the k largest logits by (value descending in the bf16 total order with NaN
//      last, index ascending);
//   2. weights in f32, every operation rounded to nearest and none fused:
//      z = (l_i - l_0) * (log2e / T), n = rint(z), f = z - n, w = poly7(f) * 2^n;
//   3. u = n53 * 2^-53; the first candidate whose running f64 sum exceeds u * total.
// One CTA per row.  The k-th largest 16-bit key is found with two 256-bin histograms (high
// byte, then low byte within the boundary bin); keys above it are collected as they are
// found, and of the keys equal to it the lowest indices are taken, which a per-thread count
// over index-contiguous runs and a block-wide prefix sum decide.
#include "common.cuh"

namespace iron {

constexpr int kSampleThreads = 1024;
constexpr int kSampleKMax = 64;

__device__ __forceinline__ uint32_t bf16_key(uint32_t bits16) {
  const uint32_t k = (bits16 & 0x8000u) ? (~bits16 & 0xffffu) : (bits16 | 0x8000u);
  return ((bits16 & 0x7fffu) > 0x7f80u) ? 0u : k;
}
__device__ __forceinline__ float key_value(uint32_t key) {
  const uint32_t bits = (key & 0x8000u) ? (key & 0x7fffu) : (~key & 0xffffu);
  return __uint_as_float(bits << 16);
}

// 2^z for z <= 0: float32, round to nearest, nothing fused (rule 2).
__device__ __forceinline__ float exp2_det(float z) {
  if (!(z >= -1000.0f)) z = -1000.0f;   // also what a NaN becomes
  const float n = rintf(z);
  const float f = __fsub_rn(z, n);
  // (ln 2)^k / k!, k = 7 .. 0
  const float c[8] = {__uint_as_float(0x377fe5feu), __uint_as_float(0x39218489u), __uint_as_float(0x3aaec3ffu), __uint_as_float(0x3c1d955bu),
                      __uint_as_float(0x3d635847u), __uint_as_float(0x3e75fdf0u), __uint_as_float(0x3f317218u), __uint_as_float(0x3f800000u)};   // as float32 bit patterns: the host's very constants
  float p = c[0];
#pragma unroll
  for (int i = 1; i < 8; ++i) p = __fadd_rn(__fmul_rn(p, f), c[i]);
  if (n < -120.0f) return 0.0f;
  return ldexpf(p, (int)n);   // exact: the result is a normal number
}

__global__ void __launch_bounds__(kSampleThreads) sample_rows_kernel(
    const __nv_bfloat16* __restrict__ logits, long long pitch, int n, const int* __restrict__ draws,
    int* __restrict__ tokens, int* __restrict__ positions, int* __restrict__ drawn, int S) {
  __shared__ unsigned int hist[256];
  __shared__ unsigned int scan[kSampleThreads / 32];
  __shared__ unsigned int s_bin, s_above, s_count;
  __shared__ unsigned long long cand[kSampleKMax];    // (key << 32) | ~index: larger = ranks earlier
  __shared__ unsigned long long sorted[kSampleKMax];
  pdl_wait();
  pdl_launch();
  const int r = blockIdx.x, tid = threadIdx.x;
  const __nv_bfloat16* row = logits + (long long)r * pitch;
  const int pos = max(0, min(positions[r], S - 1));
  const int* draw = draws + ((long long)r * S + pos) * 4;
  const float temperature = __int_as_float(draw[0]);
  int k = draw[1];
  const unsigned long long n53 = ((unsigned long long)(unsigned int)draw[3] << 32) | (unsigned int)draw[2];
  const bool greedy = !(temperature > 0.0f) || k <= 1;
  k = greedy ? 1 : min(min(k, kSampleKMax), n);

  // index-contiguous runs: thread t owns elements [t * per, (t + 1) * per)
  const int per = ((n + kSampleThreads - 1) / kSampleThreads + 7) & ~7;
  const int lo = min(n, tid * per), hi = min(n, lo + per);
  auto for_each = [&](auto&& body) {
    int i = lo;
    if ((pitch & 7) == 0)
      for (; i + 8 <= hi; i += 8) {
        const uint4 v = ld_cached(row + i);
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) { body(i + 2 * j, w[j] & 0xffffu); body(i + 2 * j + 1, w[j] >> 16); }
      }
    for (; i < hi; ++i) body(i, (uint32_t)__bfloat16_as_ushort(row[i]));
  };
  // the bin (of `shift`-ed key bytes, among keys accepted by `in`) that holds the k-th largest
  auto pick_bin = [&](int want, auto&& in, int shift) {
    for (int b = tid; b < 256; b += kSampleThreads) hist[b] = 0;
    __syncthreads();
    for_each([&](int, uint32_t bits) {
      const uint32_t key = bf16_key(bits);
      if (in(key)) atomicAdd(&hist[(key >> shift) & 0xffu], 1u);
    });
    __syncthreads();
    if (tid == 0) {
      unsigned int above = 0;
      int b = 255;
      for (; b > 0; --b) {
        if (above + hist[b] >= (unsigned int)want) break;
        above += hist[b];
      }
      s_bin = (unsigned int)b;
      s_above = above;
    }
    __syncthreads();
  };
  pick_bin(k, [](uint32_t) { return true; }, 8);
  const uint32_t hi_bin = s_bin;
  const unsigned int above_hi = s_above;
  pick_bin(k - (int)above_hi, [&](uint32_t key) { return (key >> 8) == hi_bin; }, 0);
  const uint32_t threshold = (hi_bin << 8) | s_bin;
  const unsigned int above = above_hi + s_above;           // keys strictly above the threshold (< k)
  const unsigned int need = (unsigned int)k - above;       // taken from the keys equal to it, lowest indices first

  // ties at the threshold: this thread's count, then its first rank among them
  unsigned int mine = 0;
  for_each([&](int, uint32_t bits) { mine += bf16_key(bits) == threshold; });
  unsigned int incl = mine;
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    const unsigned int o = __shfl_up_sync(0xffffffffu, incl, off);
    if ((tid & 31) >= off) incl += o;
  }
  if ((tid & 31) == 31) scan[tid >> 5] = incl;
  if (tid == 0) s_count = 0;
  __syncthreads();
  if (tid < 32) {
    unsigned int v = scan[tid];
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const unsigned int o = __shfl_up_sync(0xffffffffu, v, off);
      if (tid >= off) v += o;
    }
    scan[tid] = v;
  }
  __syncthreads();
  unsigned int tie_rank = incl - mine + ((tid >> 5) ? scan[(tid >> 5) - 1] : 0u);
  for_each([&](int i, uint32_t bits) {
    const uint32_t key = bf16_key(bits);
    bool take = key > threshold;
    if (key == threshold) take = tie_rank++ < need;
    if (take) {
      const unsigned int at = atomicAdd(&s_count, 1u);
      if (at < (unsigned int)kSampleKMax) cand[at] = ((unsigned long long)key << 32) | (uint32_t)(~(uint32_t)i);
    }
  });
  __syncthreads();
  const int kk = min((int)s_count, kSampleKMax);           // == k
  // rank by counting: value descending, index ascending
  if (tid < kk) {
    const unsigned long long me = cand[tid];
    int rank = 0;
    for (int j = 0; j < kk; ++j) rank += cand[j] > me;
    sorted[rank] = me;
  }
  __syncthreads();
  if (tid == 0) {
    int pick = 0;
    if (!greedy && kk > 1) {
      const float c = __fdiv_rn(1.4426950408889634f, temperature);
      const float l0 = key_value((uint32_t)(sorted[0] >> 32));
      double total = 0.0;
      for (int j = 0; j < kk; ++j) {
        const float z = __fmul_rn(__fsub_rn(key_value((uint32_t)(sorted[j] >> 32)), l0), c);
        total = __dadd_rn(total, (double)exp2_det(z));
      }
      const double target = __dmul_rn(__dmul_rn((double)n53, 1.1102230246251565e-16), total);
      double acc = 0.0;
      pick = kk - 1;
      for (int j = 0; j < kk; ++j) {
        const float z = __fmul_rn(__fsub_rn(key_value((uint32_t)(sorted[j] >> 32)), l0), c);
        acc = __dadd_rn(acc, (double)exp2_det(z));
        if (target < acc) { pick = j; break; }
      }
    }
    const int tok = kk > 0 ? (int)(~(uint32_t)(sorted[pick] & 0xffffffffull)) : 0;
    drawn[(size_t)r * S + pos] = tok;
    tokens[r] = tok;
    positions[r] = pos + 1;
  }
}

}  // namespace iron

using namespace iron;

extern "C" int iron_sample_k_max(void) { return kSampleKMax; }

extern "C" int iron_sample_rows_bf16(const void* logits, long long pitch, int rows, int n, const int* draws,
                                     int* tokens, int* positions, int* drawn, int S, iron_stream_t stream) {
  if (rows < 0 || n <= 0 || S <= 0 || pitch < n) return IRON_ERR_SHAPE;
  if (!logits || !draws || !tokens || !positions || !drawn) return IRON_ERR_SHAPE;
  if (!aligned16(logits)) return IRON_ERR_ALIGN;
  if (rows == 0) return IRON_OK;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)rows);
  cfg.blockDim = dim3(kSampleThreads);
  cfg.stream = (cudaStream_t)stream;
  cudaLaunchAttribute attr[1];
  fill_pdl_attr(cfg, attr);
  return cudaLaunchKernelEx(&cfg, sample_rows_kernel, (const __nv_bfloat16*)logits, pitch, n, draws, tokens, positions,
                            drawn, S) == cudaSuccess
             ? IRON_OK
             : IRON_ERR_LAUNCH;
}
