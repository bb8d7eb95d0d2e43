// One-query ("packed") attention over a KV cache, the keys split over a thread-block
// cluster.
//
// grid = (splits, kv_heads * head_chunks, batch), cluster = (splits, 1, 1), splits <= 8.
// A CTA takes one KV head, up to GQ of the query heads that share it, and a contiguous
// slice of the keys.  Inside a warp, D/8 lanes cover one key row with 128-bit loads, so a
// warp streams 32/(D/8) keys per step and a CTA a batch of UNR steps at once: all K and V
// loads of a batch are in flight together, the batch's scores are taken against the
// running maximum once (exp2 domain), and every lane group keeps (max, sum, D-slice of
// the output) per query head in registers.  Lane groups and warps merge through shuffles
// and shared memory into the CTA's partial; after one cluster barrier each CTA folds its
// share of the output elements from every CTA's partial over distributed shared memory.
// No global scratch, no atomics, no spin: the only waits are hardware barriers.
//
// When the caller promises that only the newest cache row was written by the kernel just
// before (a decode step), the first batch's loads are issued ahead of the
// programmatic-dependency wait and the newest row is re-read after it.
#include <cooperative_groups.h>

#include <cstdlib>

#include "common.cuh"

namespace cg = cooperative_groups;

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
  int stable_prefix;        // rows before the newest are not written by the previous kernel
  PrefetchHint hint;        // weights a later kernel will stream (may be empty)
};

template <int D, int GQ>
struct DecodeCfg {
  static constexpr int kWarps = (D * GQ > 1024) ? 4 : 8;
  static constexpr int kThreads = kWarps * 32;
  static constexpr int LPK = D / 8;          // lanes per key
  static constexpr int KPW = 32 / LPK;       // keys per warp step
  static constexpr int TS = KPW * kWarps;    // keys per CTA step
  static constexpr int UNR = GQ >= 8 ? 4 : 8;
};

template <int D, int GQ>
__global__ void __launch_bounds__(DecodeCfg<D, GQ>::kThreads) mha_decode_kernel(const DecodeParams p) {
  using Cfg = DecodeCfg<D, GQ>;
  constexpr int LPK = Cfg::LPK, KPW = Cfg::KPW, TS = Cfg::TS, UNR = Cfg::UNR, W = Cfg::kWarps;
  __shared__ float sm_o[W][GQ][D];
  __shared__ float sm_ml[W][GQ][2];
  __shared__ float sm_part[GQ][D + 2];  // this CTA's partial: D outputs, max, sum

  pdl_launch();
  if (threadIdx.x == 0)
    prefetch_l2_slice(p.hint, (blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x,
                      gridDim.x * gridDim.y * gridDim.z);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int split = blockIdx.x;
  const int chunks = (p.group + GQ - 1) / GQ;
  const int kvh = blockIdx.y / chunks, hc = blockIdx.y - kvh * chunks;
  const int b = blockIdx.z;
  const int h0 = kvh * p.group + hc * GQ;            // first query head of this CTA
  const int nh = min(GQ, p.group - hc * GQ);         // live heads
  const int dsel = lane % LPK, kslot = warp * KPW + lane / LPK;

  // The per-call bound was written by an earlier graph launch (or is an immediate).
  int kv_valid = p.kv_valid;
  if (p.d_kv_valid) kv_valid = p.d_kv_valid[b * p.d_kv_valid_stride] + p.kv_valid_add;
  kv_valid = max(0, min(kv_valid, p.kv_max));
  const int lo = (p.window >= 0) ? max(0, kv_valid - 1 - p.window) : 0;
  const int span = kv_valid - lo;
  const int per = (span + p.nsplit - 1) / p.nsplit;
  const int k_begin = lo + split * per;
  const int k_end = min(kv_valid, k_begin + per);

  const __nv_bfloat16* Kb = p.K + (size_t)b * p.kv_batch_stride + (size_t)kvh * p.kv_head_stride + dsel * 8;
  const __nv_bfloat16* Vb = p.V + (size_t)b * p.kv_batch_stride + (size_t)kvh * p.kv_head_stride + dsel * 8;

  uint4 kraw[UNR], vraw[UNR];
  auto load_batch = [&](int kb) {
#pragma unroll
    for (int u = 0; u < UNR; ++u) {
      const int k = kb + u * TS + kslot;
      const int kc = k < k_end ? k : max(k_end - 1, 0);
      kraw[u] = ld_cached(Kb + (size_t)kc * p.kv_seq_stride);
      vraw[u] = ld_cached(Vb + (size_t)kc * p.kv_seq_stride);
    }
  };
  const bool early = p.stable_prefix && k_begin < k_end;
  if (early) load_batch(k_begin);

  pdl_wait();

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
  if (early) {
    // the newest row was written by the kernel just before: read it again, now visible
#pragma unroll
    for (int u = 0; u < UNR; ++u) {
      const int k = k_begin + u * TS + kslot;
      if (k == kv_valid - 1) {
        kraw[u] = ld_cached(Kb + (size_t)k * p.kv_seq_stride);
        vraw[u] = ld_cached(Vb + (size_t)k * p.kv_seq_stride);
      }
    }
  }

  // The trip count is the same for every lane of the CTA (shuffles sit inside).
  for (int kb = k_begin; kb < k_end; kb += TS * UNR) {
    if (!(early && kb == k_begin)) load_batch(kb);
    float s[UNR][GQ];
#pragma unroll
    for (int u = 0; u < UNR; ++u) {
      const bool live = kb + u * TS + kslot < k_end;
      float kf[8];
      unpack8(kraw[u], kf);
#pragma unroll
      for (int h = 0; h < GQ; ++h) {
        float a = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) a = fmaf(q[h][j], kf[j], a);
#pragma unroll
        for (int off = 1; off < LPK; off <<= 1) a += __shfl_xor_sync(0xffffffffu, a, off);
        s[u][h] = (live && h < nh) ? a : -INFINITY;
      }
    }
#pragma unroll
    for (int h = 0; h < GQ; ++h) {
      float mn = m[h];
#pragma unroll
      for (int u = 0; u < UNR; ++u) mn = fmaxf(mn, s[u][h]);
      if (mn == -INFINITY) continue;  // nothing live for this lane group yet
      const float corr = exp2f(m[h] - mn);
      float pr[UNR], ps = 0.f;
#pragma unroll
      for (int u = 0; u < UNR; ++u) { pr[u] = exp2f(s[u][h] - mn); ps += pr[u]; }
      l[h] = fmaf(l[h], corr, ps);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[h][j] *= corr;
#pragma unroll
      for (int u = 0; u < UNR; ++u) {
        float vf[8];
        unpack8(vraw[u], vf);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[h][j] = fmaf(pr[u], vf[j], o[h][j]);
      }
      m[h] = mn;
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
  // ---- merge the warps of the CTA into its partial ----
  if (lane < LPK) {
#pragma unroll
    for (int h = 0; h < GQ; ++h) {
#pragma unroll
      for (int j = 0; j < 8; ++j) sm_o[warp][h][dsel * 8 + j] = o[h][j];
      if (lane == 0) { sm_ml[warp][h][0] = m[h]; sm_ml[warp][h][1] = l[h]; }
    }
  }
  __syncthreads();
  const bool direct = (p.nsplit == 1);
  for (int e = tid; e < nh * D; e += Cfg::kThreads) {
    const int h = e / D, d = e - h * D;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < W; ++w) M = fmaxf(M, sm_ml[w][h][0]);
    float L = 0.f, acc = 0.f;
#pragma unroll
    for (int w = 0; w < W; ++w) {
      const float mw = sm_ml[w][h][0];
      const float c = (mw == -INFINITY) ? 0.f : exp2f(mw - M);
      L = fmaf(sm_ml[w][h][1], c, L);
      acc = fmaf(sm_o[w][h][d], c, acc);
    }
    if (direct) {
      p.O[((size_t)b * p.H + h0 + h) * D + d] = __float2bfloat16_rn(L > 0.f ? acc / L : 0.f);
    } else {
      sm_part[h][d] = acc;
      if (d == 0) { sm_part[h][D] = M; sm_part[h][D + 1] = L; }
    }
  }
  if (direct) return;

  // ---- fold the cluster's partials: each CTA takes a slice of the output elements ----
  cg::cluster_group cluster = cg::this_cluster();
  cluster.sync();
  const int total = nh * D;
  const int slice = (total + p.nsplit - 1) / p.nsplit;
  const int e_lo = split * slice, e_hi = min(total, e_lo + slice);
  for (int e = e_lo + tid; e < e_hi; e += Cfg::kThreads) {
    const int h = e / D, d = e - h * D;
    float M = -INFINITY;
    for (int r = 0; r < p.nsplit; ++r) {
      const float* remote = cluster.map_shared_rank(&sm_part[0][0], r);
      M = fmaxf(M, remote[h * (D + 2) + D]);
    }
    float L = 0.f, acc = 0.f;
    for (int r = 0; r < p.nsplit; ++r) {
      const float* remote = cluster.map_shared_rank(&sm_part[0][0], r);
      const float ms = remote[h * (D + 2) + D];
      const float c = (ms == -INFINITY) ? 0.f : exp2f(ms - M);
      L = fmaf(remote[h * (D + 2) + D + 1], c, L);
      acc = fmaf(remote[h * (D + 2) + d], c, acc);
    }
    p.O[((size_t)b * p.H + h0 + h) * D + d] = __float2bfloat16_rn(L > 0.f ? acc / L : 0.f);
  }
  cluster.sync();  // nobody leaves while a peer may still read its shared memory
}

template <int D, int GQ>
static int launch_decode(const DecodeParams& p, int B, cudaStream_t stream) {
  using Cfg = DecodeCfg<D, GQ>;
  const int chunks = (p.group + GQ - 1) / GQ;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(p.nsplit, p.G * chunks, B);
  cfg.blockDim = dim3(Cfg::kThreads);
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = p.nsplit;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1 + pdl_attr_count();
  return cudaLaunchKernelEx(&cfg, mha_decode_kernel<D, GQ>, p) == cudaSuccess ? IRON_OK
                                                                              : IRON_ERR_LAUNCH;
}

// the resident form for a few sequences and the tensor-core kernel for batches (mha_decode_tc.cu)
int mha_decode_resident(const void* Q, const void* K, const void* V, void* O, int batch, int H, int G, int D,
                        int kv_max, long long kv_batch_stride, long long kv_seq_stride, long long kv_head_stride,
                        int kv_valid, const int* d_kv_valid, int d_kv_valid_stride, int kv_valid_add, int window,
                        float scale, int stable_prefix, cudaStream_t stream);
int mha_decode_tc(const void* Q, const void* K, const void* V, void* O, int batch, int H, int G, int D, int kv_max,
                  long long kv_batch_stride, long long kv_seq_stride, long long kv_head_stride, int kv_valid,
                  const int* d_kv_valid, int d_kv_valid_stride, int kv_valid_add, int window, float scale,
                  cudaStream_t stream);

static int decode_gq(int group) { return group >= 5 ? 8 : (group >= 3 ? 4 : (group == 2 ? 2 : 1)); }

}  // namespace iron

using namespace iron;

extern "C" int iron_mha_decode_splits(int batch, int G, int kv_len_hint) {
  // A cluster of up to eight CTAs shares one (batch, KV head): split while each CTA keeps
  // at least 64 keys and the grid stays within a few waves.
  int nsplit = 8;
  while (nsplit > 1 && kv_len_hint / nsplit < 64) nsplit >>= 1;
  while (nsplit > 1 && (long long)batch * G * nsplit > (long long)kSMs * 4) nsplit >>= 1;
  return nsplit;
}

extern "C" int iron_mha_decode_bf16(const void* Q, const void* K, const void* V, void* O,
                                    int batch, int H, int G, int D, int kv_max,
                                    long long kv_batch_stride, long long kv_seq_stride,
                                    long long kv_head_stride, int kv_valid,
                                    const int* d_kv_valid, int d_kv_valid_stride,
                                    int kv_valid_add, int window, float scale, int nsplit,
                                    int stable_prefix, iron_stream_t stream) {
  if (batch <= 0 || H <= 0 || G <= 0 || H % G) return IRON_ERR_SHAPE;
  if (D != 64 && D != 128 && D != 256) return IRON_ERR_SHAPE;
  if (kv_max <= 0 || kv_valid < 0 || kv_valid > kv_max) return IRON_ERR_SHAPE;
  if (nsplit != 1 && nsplit != 2 && nsplit != 4 && nsplit != 8) return IRON_ERR_SHAPE;
  if ((kv_batch_stride & 7) || (kv_seq_stride & 7) || (kv_head_stride & 7)) return IRON_ERR_ALIGN;
  if (!aligned16(Q) || !aligned16(K) || !aligned16(V) || !aligned16(O)) return IRON_ERR_ALIGN;
  const int group = H / G;
  // A batch of two sequences or more (at least 16 (sequence, KV head) pairs; IRON_MHA_DECODE_TC_MIN)
  // goes to the tensor-core kernel: the group's query heads are the rows of one MMA tile, and
  // the keys are split over a cluster while the pairs alone do not fill the machine.  One
  // sequence (8 pairs) measured faster on the SIMT kernel.  IRON_MHA_DECODE_TC=0 keeps the SIMT kernel.
  static const bool use_tc = [] {
    const char* e = getenv("IRON_MHA_DECODE_TC");
    return !(e && e[0] == '0');
  }();
  // fewer pairs than that: every CTA holds its share of the keys in shared memory (IRON_MHA_DECODE_RESIDENT=0
  // keeps the SIMT kernel)
  static const bool use_resident = [] {
    const char* e = getenv("IRON_MHA_DECODE_RESIDENT");
    return !(e && e[0] == '0');
  }();
  static const int tc_min = [] {
    const char* e = getenv("IRON_MHA_DECODE_TC_MIN");
    return e ? atoi(e) : 16;
  }();
  if (use_tc && use_resident && group > 1 && (long long)batch * G < tc_min) {
    const int rc = mha_decode_resident(Q, K, V, O, batch, H, G, D, kv_max, kv_batch_stride, kv_seq_stride,
                                       kv_head_stride, kv_valid, d_kv_valid, d_kv_valid_stride, kv_valid_add, window,
                                       scale, stable_prefix, (cudaStream_t)stream);
    if (rc != IRON_ERR_UNSUPPORTED) return rc;
  }
  if (use_tc && group > 1 && (long long)batch * G >= tc_min) {
    const int rc = mha_decode_tc(Q, K, V, O, batch, H, G, D, kv_max, kv_batch_stride, kv_seq_stride,
                                 kv_head_stride, kv_valid, d_kv_valid, d_kv_valid_stride, kv_valid_add, window,
                                 scale, (cudaStream_t)stream);
    if (rc != IRON_ERR_UNSUPPORTED) return rc;
  }
  // Query heads that share a KV head run in one CTA only when the grid already fills the
  // machine; a single sequence gives every query head a CTA of its own (the re-read keys
  // hit in L2) so that the per-key work spreads over all SMs.
  const int gq = ((long long)batch * G * nsplit >= 2 * kSMs) ? decode_gq(group) : 1;
  DecodeParams p = {};
  p.Q = (const __nv_bfloat16*)Q; p.K = (const __nv_bfloat16*)K; p.V = (const __nv_bfloat16*)V;
  p.O = (__nv_bfloat16*)O;
  p.kv_batch_stride = kv_batch_stride; p.kv_seq_stride = kv_seq_stride; p.kv_head_stride = kv_head_stride;
  p.H = H; p.G = G; p.group = group;
  p.kv_valid = kv_valid; p.d_kv_valid = d_kv_valid; p.d_kv_valid_stride = d_kv_valid_stride;
  p.kv_valid_add = kv_valid_add; p.kv_max = kv_max; p.window = window;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.nsplit = nsplit;
  p.stable_prefix = stable_prefix;
  p.hint = take_prefetch_hint();
  cudaStream_t s = (cudaStream_t)stream;
#define IRON_DEC(DD, QQ) if (D == DD && gq == QQ) return launch_decode<DD, QQ>(p, batch, s);
  IRON_DEC(64, 1) IRON_DEC(64, 2) IRON_DEC(64, 4) IRON_DEC(64, 8)
  IRON_DEC(128, 1) IRON_DEC(128, 2) IRON_DEC(128, 4) IRON_DEC(128, 8)
  IRON_DEC(256, 1) IRON_DEC(256, 2) IRON_DEC(256, 4) IRON_DEC(256, 8)
#undef IRON_DEC
  return IRON_ERR_UNSUPPORTED;
}
