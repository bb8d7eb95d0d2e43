// Bandwidth-bound bf16 GEMV family for sm_100a.
//
// One warp owns a *pair* of weight rows and streams them with 128-bit
// `ld.global.nc.L1::no_allocate` loads (8 independent 16-byte loads in flight per
// lane), against the activation vector staged once per CTA in shared memory.  The pair
// is what makes the fused forms free:
//   PLAIN   rows (2p, 2p+1) of one matrix                      -> GEMV
//   SWIGLU  row m of the gate matrix and row m of the up matrix -> GEMV,GEMV,SiLU,Mul
//   QKV     rows (i, i + D/2) of one head                       -> GEMV x3, RoPE, KV write
// Short-and-wide shapes (few rows, long K) split K across the warps of a CTA so that
// every SM still has tens of KB of loads outstanding.
//
// The optional prologue recomputes RMSNorm(x) per CTA (x is a few KB and L2-resident),
// with the reference's two bf16 roundings (norm, then weight).
#include <cstdlib>

#include "common.cuh"
#include "gemv_items.cuh"

namespace iron {

enum { GEMV_PLAIN = 0, GEMV_SWIGLU = 1, GEMV_QKV = 2 };

struct GemvParams {
  const __nv_bfloat16* A;     // PLAIN/QKV: the matrix; SWIGLU: gate
  const __nv_bfloat16* A2;    // SWIGLU: up
  const __nv_bfloat16* x;
  __nv_bfloat16* y;
  const __nv_bfloat16* residual;
  const __nv_bfloat16* norm_w;
  int M, K, repeat, rows;     // rows = rows actually computed (valid)
  int norm_mode;
  float eps;
  int ksplit;                 // warps sharing one row pair: 1, 2, 4 or 8
  // QKV mode
  const __nv_bfloat16* angles;
  __nv_bfloat16* k_cache;
  __nv_bfloat16* v_cache;
  const int* d_position;
  int position, H, G, D;
  PrefetchHint hint;          // weights a later kernel will stream (may be empty)
};

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kUnroll = 2;         // 256-bit loads per row per work item (4 for 128-bit loads)

template <int MODE>
__device__ __forceinline__ void pair_rows(const GemvParams& p, const __nv_bfloat16* A, int pair, int half,
                                          int& ra, int& rb, const uint4*& qa, const uint4*& qb) {
  const int K = p.K;
  const __nv_bfloat16 *pa, *pb;
  if (MODE == GEMV_PLAIN) {
    ra = 2 * pair; rb = ra + 1;
    pa = A + (size_t)ra * K;
    pb = (rb < p.rows) ? pa + K : pa;
  } else if (MODE == GEMV_SWIGLU) {
    ra = rb = pair;
    pa = A + (size_t)ra * K;
    pb = p.A2 + (size_t)ra * K;
  } else {
    const int head = pair / half, i = pair - head * half;
    ra = head * p.D + i; rb = ra + half;
    pa = A + (size_t)ra * K;
    pb = A + (size_t)rb * K;
  }
  qa = reinterpret_cast<const uint4*>(pa);
  qb = reinterpret_cast<const uint4*>(pb);
}

// The grid is persistent (at most two CTAs per SM).  A warp's first weight loads are
// issued before anything else -- they do not depend on the previous kernel -- so with
// programmatic dependent launch the weight stream of this kernel overlaps the tail of
// the one before it; the activation vector is staged (and normalised) while those
// loads are in flight, and every later item is prefetched one step ahead of its use.
template <int MODE, bool WIDE>
__global__ void __launch_bounds__(kThreads, 2) gemv_kernel(const GemvParams p) {
  extern __shared__ uint4 smem[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int K = p.K, nch = K >> 3;
  uint4* xs = smem;                                   // nch chunks of 8 bf16
  float* red = reinterpret_cast<float*>(smem + nch);  // 32 floats for block_sum
  float* part = red + 32;                             // kWarps x 2 partial sums

  pdl_launch();
  if (threadIdx.x == 0 && blockIdx.y == 0) prefetch_l2_slice(p.hint, blockIdx.x, gridDim.x);

  const int batch = blockIdx.y;
  const size_t mat = (size_t)(batch / p.repeat) * (size_t)p.M * (size_t)K;
  const __nv_bfloat16* A = p.A + mat;

  const int KS = p.ksplit;
  const int groups = kWarps / KS;       // row pairs in flight per CTA
  const int g = warp / KS, ks = warp % KS;
  constexpr int kStep = 32 * kItem;     // chunks one item covers
  const int per = ((nch + KS - 1) / KS + 1) & ~1;  // even, so 256-bit loads stay aligned
  const int ch_lo = min(nch, ks * per);
  const int ch_hi = min(nch, ch_lo + per);

  int npairs, half = 0;
  if (MODE == GEMV_PLAIN) npairs = (p.rows + 1) >> 1;
  else if (MODE == GEMV_SWIGLU) npairs = p.rows;
  else { half = p.D >> 1; npairs = p.rows >> 1; }
  const int stride = gridDim.x * groups;

  int base = blockIdx.x * groups;
  int ra = 0, rb = 0;
  const uint4 *qa = nullptr, *qb = nullptr;
  bool live = base + g < npairs;
  if (live) pair_rows<MODE>(p, A, base + g, half, ra, rb, qa, qb);
  Item cur;
  issue<WIDE>(cur, qa, qb, ch_lo, lane, ch_hi, live && ch_lo < ch_hi);

  // The activation vector is the previous kernel's output: wait for it now.
  pdl_wait();

  // ---- stage x (optionally RMS-normalised) into shared memory ----
  {
    const uint4* xg = reinterpret_cast<const uint4*>(p.x + (size_t)batch * K);
    float ss = 0.f;
    for (int i = tid; i < nch; i += kThreads) {
      uint4 v = ld_cached(xg + i);
      xs[i] = v;
      if (p.norm_mode) {
        float f[8];
        unpack8(v, f);
#pragma unroll
        for (int j = 0; j < 8; ++j) ss = fmaf(f[j], f[j], ss);
      }
    }
    if (p.norm_mode) {
      const float tot = block_sum(ss, red);
      const float inv = 1.0f / sqrtf(tot / (float)K + p.eps);
      const uint4* wg = reinterpret_cast<const uint4*>(p.norm_w);
      for (int i = tid; i < nch; i += kThreads) {
        float f[8];
        unpack8(xs[i], f);
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] = round_bf16(f[j] * inv);
        if (p.norm_mode == 2) {
          float w[8];
          unpack8(ld_cached(wg + i), w);
#pragma unroll
          for (int j = 0; j < 8; ++j) f[j] = f[j] * w[j];
        }
        xs[i] = pack8(f);
      }
    }
    __syncthreads();
  }

  for (; base < npairs; base += stride) {
    float acc0 = 0.f, acc1 = 0.f;
    // the next pair of this warp (its first item is prefetched during this pair's last)
    const bool live_n = base + stride + g < npairs;
    int ra_n = 0, rb_n = 0;
    const uint4 *qa_n = nullptr, *qb_n = nullptr;
    if (live_n) pair_rows<MODE>(p, A, base + stride + g, half, ra_n, rb_n, qa_n, qb_n);
    for (int c0 = ch_lo; c0 < ch_hi; c0 += kStep) {
      Item nxt;
      if (c0 + kStep < ch_hi) issue<WIDE>(nxt, qa, qb, c0 + kStep, lane, ch_hi, live);
      else issue<WIDE>(nxt, qa_n, qb_n, ch_lo, lane, ch_hi, live_n);
      consume<WIDE>(cur, xs, c0, lane, ch_hi, acc0, acc1);
      cur = nxt;
    }
    acc0 = warp_sum(acc0);
    acc1 = warp_sum(acc1);
    if (KS > 1) {
      if (lane == 0) { part[warp * 2] = acc0; part[warp * 2 + 1] = acc1; }
      __syncthreads();
      if (ks == 0) {
        acc0 = 0.f; acc1 = 0.f;
        for (int s = 0; s < KS; ++s) { acc0 += part[(warp + s) * 2]; acc1 += part[(warp + s) * 2 + 1]; }
      }
      __syncthreads();
    }
    if (live && ks == 0 && lane == 0) {
      if (MODE == GEMV_PLAIN) {
        __nv_bfloat16* y = p.y + (size_t)batch * p.M;
        float v0 = round_bf16(acc0), v1 = round_bf16(acc1);
        if (p.residual) {
          const __nv_bfloat16* r = p.residual + (size_t)batch * p.M;
          v0 = __fadd_rn(v0, __bfloat162float(r[ra]));
          if (rb < p.rows) v1 = __fadd_rn(v1, __bfloat162float(r[rb]));
        }
        y[ra] = __float2bfloat16_rn(v0);
        if (rb < p.rows) y[rb] = __float2bfloat16_rn(v1);
      } else if (MODE == GEMV_SWIGLU) {
        const float gate = round_bf16(acc0), up = round_bf16(acc1);
        const float act = round_bf16(silu_f32(gate));
        p.y[ra] = __float2bfloat16_rn(__fmul_rn(act, up));
      } else {
        const int pos = p.d_position ? *p.d_position : p.position;
        const int head = ra / p.D, i = ra - head * p.D;
        float x1 = round_bf16(acc0), x2 = round_bf16(acc1);
        if (head < p.H + p.G) {
          const __nv_bfloat16* ang = p.angles + (size_t)pos * p.D;
          const float c = __bfloat162float(ang[2 * i]), s = __bfloat162float(ang[2 * i + 1]);
          const float y1 = __fsub_rn(__fmul_rn(x1, c), __fmul_rn(x2, s));
          const float y2 = __fadd_rn(__fmul_rn(x2, c), __fmul_rn(x1, s));
          x1 = y1; x2 = y2;
        }
        __nv_bfloat16* dst;
        if (head < p.H) dst = p.y + (size_t)head * p.D;
        else if (head < p.H + p.G) dst = p.k_cache + ((size_t)pos * p.G + (head - p.H)) * p.D;
        else dst = p.v_cache + ((size_t)pos * p.G + (head - p.H - p.G)) * p.D;
        dst[i] = __float2bfloat16_rn(x1);
        dst[i + half] = __float2bfloat16_rn(x2);
      }
    }
    live = live_n; ra = ra_n; rb = rb_n; qa = qa_n; qb = qb_n;
  }
}

template <int MODE, bool WIDE>
static int launch_gemv_w(GemvParams& p, int npairs, int batches, cudaStream_t stream) {
  static bool configured = false;
  constexpr int kMaxSmem = 100 * 1024;
  if (!configured) {
    if (cudaFuncSetAttribute(gemv_kernel<MODE, WIDE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             kMaxSmem) != cudaSuccess)
      return IRON_ERR_LAUNCH;
    configured = true;
  }
  const int nch = p.K >> 3;
  constexpr int kStep = 32 * kItem;
  static const int per_sm = [] {
    const char* e = getenv("IRON_GEMV_CTAS_PER_SM");
    const int v = e ? atoi(e) : 2;
    return v >= 1 && v <= 2 ? v : 2;
  }();
  const int slots = per_sm * kSMs;  // resident CTAs
  // Split K across the warps of a CTA (each keeps at least one full item) while that
  // evens out the last wave: pick the split with the least idle warp-time.
  int best_ks = 1;
  double best_eff = -1.0;
  for (int ks = 1; ks <= kWarps; ks *= 2) {
    if (ks > 1 && nch / ks < kStep) break;
    const long long cta_iters = ((long long)npairs * ks + kWarps - 1) / kWarps;
    const long long waves = (cta_iters + slots - 1) / slots;
    const double eff = (double)cta_iters / (double)(waves * slots);
    const double fill = cta_iters >= slots ? 1.0 : (double)cta_iters / slots;
    const double score = cta_iters >= slots ? eff : fill * 0.9;
    if (score > best_eff + 0.02) { best_eff = score; best_ks = ks; }
  }
  p.ksplit = best_ks;
  p.hint = take_prefetch_hint();
  const int groups = kWarps / best_ks;
  const long long cta_iters = (npairs + groups - 1) / groups;
  const long long waves = (cta_iters + slots - 1) / slots;
  int ctas = (int)((cta_iters + waves - 1) / waves);  // equal work per CTA
  if (batches > 1) ctas = (int)(cta_iters < slots ? cta_iters : slots);
  ctas = ctas < 1 ? 1 : ctas;
  const size_t smem = (size_t)nch * 16 + (32 + 2 * kWarps) * sizeof(float);
  if (smem > (size_t)kMaxSmem) return IRON_ERR_SHAPE;

  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(ctas, batches, 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  fill_pdl_attr(cfg, attr);
  if (cudaLaunchKernelEx(&cfg, gemv_kernel<MODE, WIDE>, p) != cudaSuccess) return IRON_ERR_LAUNCH;
  return IRON_OK;
}

static bool aligned32(const void* q) { return (reinterpret_cast<uintptr_t>(q) & 31u) == 0; }

template <int MODE>
static int launch_gemv(GemvParams& p, int npairs, int batches, cudaStream_t stream) {
  const bool wide = (p.K % 16 == 0) && aligned32(p.A) && (MODE != GEMV_SWIGLU || aligned32(p.A2));
  return wide ? launch_gemv_w<MODE, true>(p, npairs, batches, stream)
              : launch_gemv_w<MODE, false>(p, npairs, batches, stream);
}

static int check_common(const void* A, const void* x, const void* y, int M, int K) {
  if (M <= 0 || K <= 0 || (K & 7) || K > 49152) return IRON_ERR_SHAPE;
  if (!aligned16(A) || !aligned16(x) || !aligned16(y)) return IRON_ERR_ALIGN;
  return IRON_OK;
}

}  // namespace iron

using namespace iron;

extern "C" int iron_gemv_bf16(const void* A, const void* x, void* y, int M, int K, int batches,
                              int repeat, int valid_rows, int norm_mode,
                              const void* norm_weight, float eps, const void* residual,
                              iron_stream_t stream) {
  int rc = check_common(A, x, y, M, K);
  if (rc) return rc;
  if (batches <= 0 || repeat <= 0 || batches % repeat) return IRON_ERR_SHAPE;
  if (valid_rows < 0 || valid_rows > M) return IRON_ERR_SHAPE;
  if (norm_mode < 0 || norm_mode > 2 || (norm_mode == 2 && !norm_weight)) return IRON_ERR_SHAPE;
  if (norm_mode == 2 && !aligned16(norm_weight)) return IRON_ERR_ALIGN;
  if (valid_rows == 0) return IRON_OK;
  GemvParams p = {};
  p.A = (const __nv_bfloat16*)A; p.x = (const __nv_bfloat16*)x; p.y = (__nv_bfloat16*)y;
  p.residual = (const __nv_bfloat16*)residual; p.norm_w = (const __nv_bfloat16*)norm_weight;
  p.M = M; p.K = K; p.repeat = repeat; p.rows = valid_rows; p.norm_mode = norm_mode; p.eps = eps;
  return launch_gemv<GEMV_PLAIN>(p, (valid_rows + 1) / 2, batches, (cudaStream_t)stream);
}

extern "C" int iron_gemv_swiglu_bf16(const void* Wg, const void* Wu, const void* x, void* y,
                                     int M, int K, int norm_mode, const void* norm_weight,
                                     float eps, iron_stream_t stream) {
  int rc = check_common(Wg, x, y, M, K);
  if (rc) return rc;
  if (!aligned16(Wu)) return IRON_ERR_ALIGN;
  if (norm_mode < 0 || norm_mode > 2 || (norm_mode == 2 && !norm_weight)) return IRON_ERR_SHAPE;
  GemvParams p = {};
  p.A = (const __nv_bfloat16*)Wg; p.A2 = (const __nv_bfloat16*)Wu;
  p.x = (const __nv_bfloat16*)x; p.y = (__nv_bfloat16*)y;
  p.norm_w = (const __nv_bfloat16*)norm_weight;
  p.M = M; p.K = K; p.repeat = 1; p.rows = M; p.norm_mode = norm_mode; p.eps = eps;
  return launch_gemv<GEMV_SWIGLU>(p, M, 1, (cudaStream_t)stream);
}

extern "C" int iron_decode_qkv_rope_bf16(const void* Wqkv, const void* x, int K, int norm_mode,
                                         const void* norm_weight, float eps, const void* angles,
                                         int position, const int* d_position, void* q_out,
                                         void* k_cache, void* v_cache, int H, int G, int D,
                                         iron_stream_t stream) {
  if (H <= 0 || G <= 0 || D <= 0 || (D & 15)) return IRON_ERR_SHAPE;
  const int M = (H + 2 * G) * D;
  int rc = check_common(Wqkv, x, q_out, M, K);
  if (rc) return rc;
  if (!angles || !k_cache || !v_cache) return IRON_ERR_SHAPE;
  if (norm_mode < 0 || norm_mode > 2 || (norm_mode == 2 && !norm_weight)) return IRON_ERR_SHAPE;
  if (!d_position && position < 0) return IRON_ERR_SHAPE;
  GemvParams p = {};
  p.A = (const __nv_bfloat16*)Wqkv; p.x = (const __nv_bfloat16*)x; p.y = (__nv_bfloat16*)q_out;
  p.norm_w = (const __nv_bfloat16*)norm_weight;
  p.M = M; p.K = K; p.repeat = 1; p.rows = M; p.norm_mode = norm_mode; p.eps = eps;
  p.angles = (const __nv_bfloat16*)angles;
  p.k_cache = (__nv_bfloat16*)k_cache; p.v_cache = (__nv_bfloat16*)v_cache;
  p.d_position = d_position; p.position = position; p.H = H; p.G = G; p.D = D;
  return launch_gemv<GEMV_QKV>(p, M / 2, 1, (cudaStream_t)stream);
}
