// The two row-wise kernels a *batched* decode step needs beside the GEMMs and the packed
// attention: every row of the batch is another sequence, at its own position, with its own
// KV cache.
//
//   rope_kv_scatter  RoPE on q and k of each row with the angle row of that row's position,
//                    q to a dense (rows, H, D) buffer, k and v into row `position` of that
//                    sequence's caches.
//   argmax_rows      greedy draw per row: the first index of the maximum goes to
//                    drawn[row][position], becomes the row's next token, and the row's
//                    position advances -- the carried (token, position) of the one-sequence
//                    step, once per sequence.
#include "common.cuh"

namespace iron {

// One thread per 8 rotation pairs (or 16 copied elements) of one head of one row.
__global__ void __launch_bounds__(256) rope_kv_scatter_kernel(
    const __nv_bfloat16* __restrict__ qkv, long long pitch, const __nv_bfloat16* __restrict__ angles,
    __nv_bfloat16* __restrict__ q_out, __nv_bfloat16* __restrict__ k_cache, __nv_bfloat16* __restrict__ v_cache,
    long long kv_batch_stride, int rows, const int* __restrict__ d_positions, int H, int G, int D, int S) {
  pdl_wait();
  pdl_launch();
  const int half = D >> 1, per_head = half >> 3, heads = H + 2 * G;
  const long long total = (long long)rows * heads * per_head;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int pg = (int)(idx % per_head);
    const int hh = (int)((idx / per_head) % heads);
    const int r = (int)(idx / ((long long)per_head * heads));
    const int pos = max(0, min(d_positions[r], S - 1));
    const int i0 = pg * 8;
    const __nv_bfloat16* src = qkv + (long long)r * pitch + (long long)hh * D;
    float a[8], b[8];
    unpack8(ld_cached(src + i0), a);
    unpack8(ld_cached(src + half + i0), b);
    if (hh < H + G) {
      const __nv_bfloat16* ar = angles + (size_t)pos * D;
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
    if (hh < H) dst = q_out + ((size_t)r * H + hh) * D;
    else if (hh < H + G) dst = k_cache + (size_t)r * kv_batch_stride + ((size_t)pos * G + (hh - H)) * D;
    else dst = v_cache + (size_t)r * kv_batch_stride + ((size_t)pos * G + (hh - H - G)) * D;
    *reinterpret_cast<uint4*>(dst + i0) = pack8(a);
    *reinterpret_cast<uint4*>(dst + half + i0) = pack8(b);
  }
}

__device__ __forceinline__ unsigned long long row_key(float v, int idx) {
  uint32_t u = __float_as_uint(v);
  u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
  if (v != v) u = 0;
  return ((unsigned long long)u << 32) | (uint32_t)(~(uint32_t)idx);
}

// One CTA per row.
__global__ void __launch_bounds__(1024) argmax_rows_kernel(const __nv_bfloat16* __restrict__ logits, long long pitch,
                                                           int n, int* __restrict__ tokens, int* __restrict__ positions,
                                                           int* __restrict__ drawn, int S) {
  __shared__ unsigned long long part[32];
  pdl_wait();
  pdl_launch();
  const int r = blockIdx.x;
  const __nv_bfloat16* row = logits + (long long)r * pitch;
  unsigned long long best = 0ull;
  const int nch = n >> 3;
  for (int i = threadIdx.x; i < nch; i += blockDim.x) {
    float f[8];
    unpack8(ld_stream(reinterpret_cast<const uint4*>(row) + i), f);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const unsigned long long k = row_key(f[j], i * 8 + j);
      best = k > best ? k : best;
    }
  }
  for (int i = (nch << 3) + threadIdx.x; i < n; i += blockDim.x) {
    const unsigned long long k = row_key(__bfloat162float(row[i]), i);
    best = k > best ? k : best;
  }
#pragma unroll
  for (int off = 16; off; off >>= 1) {
    const unsigned long long o = __shfl_xor_sync(0xffffffffu, best, off);
    best = o > best ? o : best;
  }
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = best;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < (int)(blockDim.x >> 5); ++w) best = part[w] > best ? part[w] : best;
    const int tok = (int)(~(uint32_t)(best & 0xffffffffull));
    const int pos = max(0, min(positions[r], S - 1));
    drawn[(size_t)r * S + pos] = tok;
    tokens[r] = tok;
    positions[r] = pos + 1;
  }
}

}  // namespace iron

using namespace iron;

extern "C" int iron_rope_kv_scatter_bf16(const void* qkv, long long pitch, const void* angles, void* q_out,
                                         void* k_cache, void* v_cache, long long kv_batch_stride, int rows,
                                         const int* d_positions, int H, int G, int D, int S,
                                         iron_stream_t stream) {
  if (rows < 0 || H <= 0 || G <= 0 || D <= 0 || (D & 15) || S <= 0) return IRON_ERR_SHAPE;
  if (!qkv || !angles || !q_out || !k_cache || !v_cache || !d_positions) return IRON_ERR_SHAPE;
  if (pitch < (long long)(H + 2 * G) * D || (pitch & 7) || (kv_batch_stride & 7)) return IRON_ERR_SHAPE;
  if (!aligned16(qkv) || !aligned16(angles) || !aligned16(q_out) || !aligned16(k_cache) || !aligned16(v_cache))
    return IRON_ERR_ALIGN;
  if (rows == 0) return IRON_OK;
  const long long items = (long long)rows * (H + 2 * G) * (D / 16);
  long long blocks = (items + 255) / 256;
  blocks = blocks < 1 ? 1 : (blocks > 4 * kSMs ? 4 * kSMs : blocks);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)blocks);
  cfg.blockDim = dim3(256);
  cfg.stream = (cudaStream_t)stream;
  cudaLaunchAttribute attr[1];
  fill_pdl_attr(cfg, attr);
  return cudaLaunchKernelEx(&cfg, rope_kv_scatter_kernel, (const __nv_bfloat16*)qkv, pitch,
                            (const __nv_bfloat16*)angles, (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_cache,
                            (__nv_bfloat16*)v_cache, kv_batch_stride, rows, d_positions, H, G, D, S) == cudaSuccess
             ? IRON_OK
             : IRON_ERR_LAUNCH;
}

extern "C" int iron_argmax_rows_bf16(const void* logits, long long pitch, int rows, int n, int* tokens,
                                     int* positions, int* drawn, int S, iron_stream_t stream) {
  if (rows < 0 || n <= 0 || S <= 0 || pitch < n || (pitch & 7)) return IRON_ERR_SHAPE;
  if (!logits || !tokens || !positions || !drawn) return IRON_ERR_SHAPE;
  if (!aligned16(logits)) return IRON_ERR_ALIGN;
  if (rows == 0) return IRON_OK;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)rows);
  cfg.blockDim = dim3(1024);
  cfg.stream = (cudaStream_t)stream;
  cudaLaunchAttribute attr[1];
  fill_pdl_attr(cfg, attr);
  return cudaLaunchKernelEx(&cfg, argmax_rows_kernel, (const __nv_bfloat16*)logits, pitch, n, tokens, positions,
                            drawn, S) == cudaSuccess
             ? IRON_OK
             : IRON_ERR_LAUNCH;
}
