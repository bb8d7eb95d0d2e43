// One-query ("packed") attention over a KV cache, split over the keys.
//
// grid = (splits, kv_heads * head_chunks, batch).  A CTA takes one KV head, up to GQ of
// the query heads that share it, and a contiguous slice of the keys.  Inside a warp,
// D/8 lanes cover one key row with 128-bit loads (K and V of the same key issued
// together), so a warp streams 32/(D/8) keys per step; every lane group keeps an online
// softmax (running max, sum and D-slice of the output, log2 domain) per query head in
// registers.  Lane groups and warps are merged by shuffles and shared memory, the CTA's
// partial goes to the workspace, and the last CTA of a (batch, head chunk) to arrive
// merges the partials and writes O -- nobody waits on anybody, so nothing can hang.
#include "common.cuh"

namespace iron {

struct DecodeParams {
  const __nv_bfloat16* Q;   // (B, H, D)
  const __nv_bfloat16* K;
  const __nv_bfloat16* V;
  __nv_bfloat16* O;         // (B, H, D)
  long long kv_batch_stride, kv_seq_stride, kv_head_stride;  // elements
  int H, G, group;          // group = H / G
  int kv_valid;
  const int* d_kv_valid;
  int d_kv_valid_stride;    // 0: one value for every batch entry; 1: one per entry
  int kv_valid_add;         // added to the device value (position -> position + 1)
  int kv_max;               // the cache's rows: device values are clamped to it
  int window;               // < 0: none
  float scale_log2;         // scale * log2(e)
  int nsplit;
  float* partial;           // (B, H, nsplit, D + 2)
  unsigned int* counters;   // (B, G * head_chunks)
};

constexpr int kDecThreads = 128;
constexpr int kDecWarps = kDecThreads / 32;

template <int D, int GQ>
__global__ void __launch_bounds__(kDecThreads) mha_decode_kernel(const DecodeParams p) {
  constexpr int LPK = D / 8;        // lanes per key
  constexpr int KPW = 32 / LPK;     // keys per warp step
  constexpr int TS = KPW * kDecWarps;
  __shared__ float sm_o[kDecWarps][GQ][D];
  __shared__ float sm_ml[kDecWarps][GQ][2];
  __shared__ bool sm_last;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int split = blockIdx.x;
  const int chunks = (p.group + GQ - 1) / GQ;
  const int kvh = blockIdx.y / chunks, hc = blockIdx.y - kvh * chunks;
  const int b = blockIdx.z;
  const int h0 = kvh * p.group + hc * GQ;            // first query head of this CTA
  const int nh = min(GQ, p.group - hc * GQ);         // live heads
  const int dsel = lane % LPK, kslot = warp * KPW + lane / LPK;

  pdl_wait();
  pdl_launch();

  int kv_valid = p.kv_valid;
  if (p.d_kv_valid) kv_valid = p.d_kv_valid[b * p.d_kv_valid_stride] + p.kv_valid_add;
  kv_valid = max(0, min(kv_valid, p.kv_max));
  const int lo = (p.window >= 0) ? max(0, kv_valid - 1 - p.window) : 0;
  const int span = kv_valid - lo;
  const int per = (span + p.nsplit - 1) / p.nsplit;
  const int k_begin = lo + split * per;
  const int k_end = min(kv_valid, k_begin + per);

  float q[GQ][8], o[GQ][8], m[GQ], l[GQ];
#pragma unroll
  for (int h = 0; h < GQ; ++h) {
    m[h] = -INFINITY; l[h] = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) { o[h][j] = 0.f; q[h][j] = 0.f; }
    if (h < nh) {
      unpack8(ld_cached(p.Q + ((size_t)b * p.H + h0 + h) * D + dsel * 8), q[h]);
#pragma unroll
      for (int j = 0; j < 8; ++j) q[h][j] *= p.scale_log2;
    }
  }

  const __nv_bfloat16* Kb = p.K + (size_t)b * p.kv_batch_stride + (size_t)kvh * p.kv_head_stride + dsel * 8;
  const __nv_bfloat16* Vb = p.V + (size_t)b * p.kv_batch_stride + (size_t)kvh * p.kv_head_stride + dsel * 8;
  // The trip count is the same for every lane of the CTA (shuffles sit inside); a lane
  // group past the end re-reads the last key and skips the update.
#pragma unroll 2
  for (int kb = k_begin; kb < k_end; kb += TS) {
    const int k = kb + kslot;
    const bool live = k < k_end;
    const int kc = live ? k : (k_end - 1);
    const uint4 kraw = ld_cached(Kb + (size_t)kc * p.kv_seq_stride);
    const uint4 vraw = ld_cached(Vb + (size_t)kc * p.kv_seq_stride);
    float kf[8], vf[8];
    unpack8(kraw, kf);
    unpack8(vraw, vf);
#pragma unroll
    for (int h = 0; h < GQ; ++h) {
      float s = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) s = fmaf(q[h][j], kf[j], s);
#pragma unroll
      for (int off = 1; off < LPK; off <<= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
      if (live && h < nh) {
        const float mn = fmaxf(m[h], s);
        const float corr = exp2f(m[h] - mn);
        const float pr = exp2f(s - mn);
        l[h] = fmaf(l[h], corr, pr);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[h][j] = fmaf(o[h][j], corr, pr * vf[j]);
        m[h] = mn;
      }
    }
  }

  // ---- merge the lane groups of a warp ----
#pragma unroll
  for (int off = LPK; off < 32; off <<= 1) {
#pragma unroll
    for (int h = 0; h < GQ; ++h) {
      const float mo = __shfl_xor_sync(0xffffffffu, m[h], off);
      const float lo2 = __shfl_xor_sync(0xffffffffu, l[h], off);
      const float mn = fmaxf(m[h], mo);
      const float ca = (m[h] == -INFINITY) ? 0.f : exp2f(m[h] - mn);
      const float cb = (mo == -INFINITY) ? 0.f : exp2f(mo - mn);
      l[h] = l[h] * ca + lo2 * cb;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float oo = __shfl_xor_sync(0xffffffffu, o[h][j], off);
        o[h][j] = o[h][j] * ca + oo * cb;
      }
      m[h] = mn;
    }
  }
  // ---- merge the warps of the CTA ----
  if (lane < LPK) {
#pragma unroll
    for (int h = 0; h < GQ; ++h) {
#pragma unroll
      for (int j = 0; j < 8; ++j) sm_o[warp][h][dsel * 8 + j] = o[h][j];
      if (lane == 0) { sm_ml[warp][h][0] = m[h]; sm_ml[warp][h][1] = l[h]; }
    }
  }
  __syncthreads();
  // thread t owns output element (h, d) for t = h * D + d, strided over the CTA
  const bool direct = (p.nsplit == 1);
  for (int e = tid; e < nh * D; e += kDecThreads) {
    const int h = e / D, d = e - h * D;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < kDecWarps; ++w) M = fmaxf(M, sm_ml[w][h][0]);
    float L = 0.f, acc = 0.f;
#pragma unroll
    for (int w = 0; w < kDecWarps; ++w) {
      const float mw = sm_ml[w][h][0];
      const float c = (mw == -INFINITY) ? 0.f : exp2f(mw - M);
      L = fmaf(sm_ml[w][h][1], c, L);
      acc = fmaf(sm_o[w][h][d], c, acc);
    }
    if (direct) {
      p.O[((size_t)b * p.H + h0 + h) * D + d] = __float2bfloat16_rn(L > 0.f ? acc / L : 0.f);
    } else {
      float* dst = p.partial + (((size_t)b * p.H + h0 + h) * p.nsplit + split) * (D + 2);
      dst[d] = acc;
      if (d == 0) { dst[D] = M; dst[D + 1] = L; }
    }
  }
  if (direct) return;

  // ---- last CTA of this (batch, head chunk) merges the splits ----
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    unsigned int* ctr = p.counters + (size_t)b * gridDim.y + blockIdx.y;
    const unsigned int arrived = atomicAdd(ctr, 1u);
    sm_last = (arrived == (unsigned int)p.nsplit - 1);
    if (sm_last) *ctr = 0;  // ready for the next launch
  }
  __syncthreads();
  if (!sm_last) return;
  __threadfence();
  for (int e = tid; e < nh * D; e += kDecThreads) {
    const int h = e / D, d = e - h * D;
    const volatile float* src = p.partial + ((size_t)b * p.H + h0 + h) * p.nsplit * (D + 2);
    float M = -INFINITY;
    for (int s = 0; s < p.nsplit; ++s) M = fmaxf(M, src[s * (D + 2) + D]);
    float L = 0.f, acc = 0.f;
    for (int s = 0; s < p.nsplit; ++s) {
      const float ms = src[s * (D + 2) + D];
      const float c = (ms == -INFINITY) ? 0.f : exp2f(ms - M);
      L = fmaf(src[s * (D + 2) + D + 1], c, L);
      acc = fmaf(src[s * (D + 2) + d], c, acc);
    }
    p.O[((size_t)b * p.H + h0 + h) * D + d] = __float2bfloat16_rn(L > 0.f ? acc / L : 0.f);
  }
}

template <int D, int GQ>
static int launch_decode(const DecodeParams& p, int B, cudaStream_t stream) {
  const int chunks = (p.group + GQ - 1) / GQ;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(p.nsplit, p.G * chunks, B);
  cfg.blockDim = dim3(kDecThreads);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, mha_decode_kernel<D, GQ>, p) == cudaSuccess ? IRON_OK
                                                                              : IRON_ERR_LAUNCH;
}

static int decode_gq(int group) { return group >= 5 ? 8 : (group >= 3 ? 4 : (group == 2 ? 2 : 1)); }
static size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

}  // namespace iron

using namespace iron;

extern "C" int iron_mha_decode_splits(int batch, int G, int kv_len_hint) {
  // about 32 keys per warp-step-quartet keeps a CTA at two to four iterations; stop
  // splitting once the grid covers the machine eight times over.
  int nsplit = (kv_len_hint + 63) / 64;
  if (nsplit < 1) nsplit = 1;
  if (nsplit > 64) nsplit = 64;
  while (nsplit > 1 && (long long)batch * G * nsplit > (long long)kSMs * 8) nsplit >>= 1;
  return nsplit;
}

extern "C" size_t iron_mha_decode_workspace_bytes(int batch, int H, int G, int D, int nsplit) {
  const int group = H / (G > 0 ? G : 1);
  const int gq = decode_gq(group);
  const int chunks = (group + gq - 1) / gq;
  const size_t counters = align_up((size_t)batch * G * chunks * sizeof(unsigned int), 256);
  const size_t partial = (size_t)batch * H * nsplit * (D + 2) * sizeof(float);
  return counters + align_up(partial, 256);
}

extern "C" int iron_mha_decode_bf16(const void* Q, const void* K, const void* V, void* O,
                                    int batch, int H, int G, int D, int kv_max,
                                    long long kv_batch_stride, long long kv_seq_stride,
                                    long long kv_head_stride, int kv_valid,
                                    const int* d_kv_valid, int d_kv_valid_stride,
                                    int kv_valid_add, int window, float scale, int nsplit,
                                    void* workspace, size_t workspace_bytes,
                                    iron_stream_t stream) {
  if (batch <= 0 || H <= 0 || G <= 0 || H % G) return IRON_ERR_SHAPE;
  if (D != 64 && D != 128 && D != 256) return IRON_ERR_SHAPE;
  if (kv_max <= 0 || kv_valid < 0 || kv_valid > kv_max) return IRON_ERR_SHAPE;
  if (nsplit < 1 || nsplit > 1024) return IRON_ERR_SHAPE;
  if ((kv_batch_stride & 7) || (kv_seq_stride & 7) || (kv_head_stride & 7)) return IRON_ERR_ALIGN;
  if (!aligned16(Q) || !aligned16(K) || !aligned16(V) || !aligned16(O)) return IRON_ERR_ALIGN;
  const int group = H / G;
  const int gq = decode_gq(group);
  const int chunks = (group + gq - 1) / gq;
  DecodeParams p = {};
  p.Q = (const __nv_bfloat16*)Q; p.K = (const __nv_bfloat16*)K; p.V = (const __nv_bfloat16*)V;
  p.O = (__nv_bfloat16*)O;
  p.kv_batch_stride = kv_batch_stride; p.kv_seq_stride = kv_seq_stride; p.kv_head_stride = kv_head_stride;
  p.H = H; p.G = G; p.group = group;
  p.kv_valid = kv_valid; p.d_kv_valid = d_kv_valid; p.d_kv_valid_stride = d_kv_valid_stride;
  p.kv_valid_add = kv_valid_add; p.kv_max = kv_max; p.window = window;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.nsplit = nsplit;
  if (nsplit > 1) {
    if (!workspace || (reinterpret_cast<uintptr_t>(workspace) & 255)) return IRON_ERR_ALIGN;
    if (workspace_bytes < iron_mha_decode_workspace_bytes(batch, H, G, D, nsplit)) return IRON_ERR_WORKSPACE;
    const size_t counters = align_up((size_t)batch * G * chunks * sizeof(unsigned int), 256);
    p.counters = (unsigned int*)workspace;
    p.partial = (float*)((char*)workspace + counters);
  }
  cudaStream_t s = (cudaStream_t)stream;
#define IRON_DEC(DD, QQ) if (D == DD && gq == QQ) return launch_decode<DD, QQ>(p, batch, s);
  IRON_DEC(64, 1) IRON_DEC(64, 2) IRON_DEC(64, 4) IRON_DEC(64, 8)
  IRON_DEC(128, 1) IRON_DEC(128, 2) IRON_DEC(128, 4) IRON_DEC(128, 8)
  IRON_DEC(256, 1) IRON_DEC(256, 2) IRON_DEC(256, 4) IRON_DEC(256, 8)
#undef IRON_DEC
  return IRON_ERR_UNSUPPORTED;
}
