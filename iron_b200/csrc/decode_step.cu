// One decode step of a Llama-architecture model as ONE persistent kernel.
//
// The five kernels a layer takes when launched separately (QKV+RoPE+cache write,
// attention, o_proj, gate/up+SwiGLU, down_proj) each pay a few microseconds of dependent
// launch and ramp-up latency, which at batch 1 is as long as the weight streaming itself.
// Here the whole step -- every layer, the final norm, the head and the greedy draw -- runs
// as phases of one cooperative grid (two CTAs per SM), separated by a grid-wide barrier
// that is split in two: a CTA *arrives* when its part of a phase is stored, then issues
// the first weight loads of the next phase, and only then *waits* for everyone's arrival.
// The weight stream therefore never stops at a phase boundary.
//
// The barrier is a monotonically increasing counter in global memory (zeroed by a memset
// node ahead of the kernel).  The launch is cooperative, so every CTA is resident and the
// barrier cannot deadlock on scheduling; every spin is still bounded by a wall-clock
// limit, after which the CTA records IRON_ERR_TIMEOUT in the status word and every CTA
// leaves.  Arithmetic and roundings are those of the separate kernels.
#include <cuda.h>

#include "common.cuh"
#include "gemv_items.cuh"

namespace iron {

constexpr int kStepThreads = 256;
constexpr int kStepWarps = kStepThreads / 32;
constexpr unsigned long long kStepWaitNs = 2000000000ull;  // 2 s

struct StepLayer {
  const __nv_bfloat16 *ln1, *wqkv, *wo, *ln2, *wg, *wu, *wd;
  __nv_bfloat16 *k, *v;
};

struct PhasePlan {
  int ksplit, ctas;
};

struct StepParams {
  const StepLayer* layers;  // device array of L entries
  int L, E, F, H, G, D, V, S;
  const __nv_bfloat16 *embed, *head, *final_norm, *angles;
  float eps, scale_log2;
  int window;
  int* values;              // [token, position]; updated at the end
  int* drawn;               // (S)
  __nv_bfloat16 *xa, *xb, *q, *act, *logits;
  float* att_part;          // (H, nsplit, D + 2)
  int nsplit;
  unsigned int* barrier;
  unsigned long long* best; // one partial argmax key per CTA
  int* status;
  PhasePlan qkv, o, swiglu, down, headp;
};

// ---- grid barrier, split into arrive and wait ----------------------------------------
__device__ __forceinline__ unsigned int ld_acquire(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.gpu.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned long long step_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void grid_arrive(unsigned int* bar) {
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    atomicAdd(bar, 1u);
  }
}
// All CTAs have arrived `epoch` times.  Returns false when the step is being abandoned.
__device__ __forceinline__ bool grid_wait(unsigned int* bar, unsigned int epoch, int* status, int* s_abort) {
  if (threadIdx.x == 0) {
    const unsigned int target = epoch * gridDim.x;
    if (ld_acquire(bar) < target) {
      const unsigned long long t0 = step_ns();
      for (unsigned int it = 1;; ++it) {
        if (ld_acquire(bar) >= target) break;
        if ((it & 255u) == 0) {
          if (*reinterpret_cast<volatile int*>(status) != 0) { *s_abort = 1; break; }
          if (step_ns() - t0 > kStepWaitNs) {
            *reinterpret_cast<volatile int*>(status) = IRON_ERR_TIMEOUT;
            *s_abort = 1;
            break;
          }
        }
      }
    }
  }
  __syncthreads();
  return *reinterpret_cast<volatile int*>(s_abort) == 0;
}

// ---- argmax key: (value, lower index first) as one 64-bit maximum --------------------
__device__ __forceinline__ unsigned long long step_key(float v, int idx) {
  uint32_t u = __float_as_uint(v);
  u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
  if (v != v) u = 0;
  return ((unsigned long long)u << 32) | (uint32_t)(~(uint32_t)idx);
}
__device__ __forceinline__ unsigned long long step_max(unsigned long long a, unsigned long long b) {
  return a > b ? a : b;
}

// Data another CTA wrote earlier in this kernel is read through L2 (L1 is not coherent).
__device__ __forceinline__ float ldcg_bf16(const __nv_bfloat16* p) {
  return __uint_as_float((uint32_t)__ldcg(reinterpret_cast<const unsigned short*>(p)) << 16);
}

enum { PH_PLAIN = 0, PH_SWIGLU = 1, PH_QKV = 2 };
enum { ST_VECTOR = 0, ST_ATTENTION = 1 };

struct PhaseArgs {
  const __nv_bfloat16 *A, *A2;       // weights (A2: the up matrix of SWIGLU)
  const __nv_bfloat16* x;            // ST_VECTOR: the activation vector
  const __nv_bfloat16* norm_w;       // non-null: RMSNorm(x) * norm_w is staged
  const __nv_bfloat16* residual;     // PLAIN: added after the rounding
  __nv_bfloat16* y;
  int rows, K;                       // output rows, reduction length
  PhasePlan plan;
  int stage;                         // ST_*
  int track_best;                    // PLAIN: keep the greedy maximum of the rows written
  // QKV
  __nv_bfloat16 *k_cache, *v_cache;
  int pos;
};

struct StepShared {
  int abort;
  float red[32];
  float part[2 * kStepWarps];
  unsigned long long best[kStepWarps];
  float att_ml[kStepWarps][2];
};

// One GEMV-shaped phase.  `xs` holds K/8 16-byte chunks of the staged activation vector.
// The CTA's first weight item is issued before the wait for the previous phase.
template <int MODE, bool WIDE>
__device__ __forceinline__ bool gemv_phase(const StepParams& sp, const PhaseArgs& a, uint4* xs, StepShared& sh,
                                           unsigned int& epoch, unsigned long long& best) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int K = a.K, nch = K >> 3;
  const int KS = a.plan.ksplit;
  const int groups = kStepWarps / KS;
  const int g = warp / KS, ks = warp % KS;
  constexpr int kStep = 32 * kItem;
  const int per = ((nch + KS - 1) / KS + 1) & ~1;
  const int ch_lo = min(nch, ks * per), ch_hi = min(nch, ch_lo + per);
  const int half = sp.D >> 1;
  int npairs;
  if (MODE == PH_PLAIN) npairs = (a.rows + 1) >> 1;
  else if (MODE == PH_SWIGLU) npairs = a.rows;
  else npairs = a.rows >> 1;
  const bool active = (int)blockIdx.x < a.plan.ctas;
  const int stride = a.plan.ctas * groups;

  auto rows_of = [&](int pair, int& ra, int& rb, const uint4*& qa, const uint4*& qb) {
    const __nv_bfloat16 *pa, *pb;
    if (MODE == PH_PLAIN) {
      ra = 2 * pair; rb = ra + 1;
      pa = a.A + (size_t)ra * K;
      pb = (rb < a.rows) ? pa + K : pa;
    } else if (MODE == PH_SWIGLU) {
      ra = rb = pair;
      pa = a.A + (size_t)ra * K;
      pb = a.A2 + (size_t)ra * K;
    } else {
      const int head = pair / half, i = pair - head * half;
      ra = head * sp.D + i; rb = ra + half;
      pa = a.A + (size_t)ra * K;
      pb = a.A + (size_t)rb * K;
    }
    qa = reinterpret_cast<const uint4*>(pa);
    qb = reinterpret_cast<const uint4*>(pb);
  };

  int base = blockIdx.x * groups;
  int ra = 0, rb = 0;
  const uint4 *qa = nullptr, *qb = nullptr;
  bool live = active && base + g < npairs;
  if (live) rows_of(base + g, ra, rb, qa, qb);
  Item cur;
  issue<WIDE>(cur, qa, qb, ch_lo, lane, ch_hi, live && ch_lo < ch_hi);

  // everything the previous phase wrote is visible after this
  if (!grid_wait(sp.barrier, epoch, sp.status, &sh.abort)) return false;

  if (active) {
    // ---- stage the activation vector ----
    if (a.stage == ST_VECTOR) {
      const uint4* xg = reinterpret_cast<const uint4*>(a.x);
      float ss = 0.f;
      for (int i = tid; i < nch; i += kStepThreads) {
        const uint4 v = __ldcg(xg + i);
        xs[i] = v;
        if (a.norm_w) {
          float f[8];
          unpack8(v, f);
#pragma unroll
          for (int j = 0; j < 8; ++j) ss = fmaf(f[j], f[j], ss);
        }
      }
      if (a.norm_w) {
        const float tot = block_sum(ss, sh.red);
        const float inv = 1.0f / sqrtf(tot / (float)K + sp.eps);
        const uint4* wg = reinterpret_cast<const uint4*>(a.norm_w);
        for (int i = tid; i < nch; i += kStepThreads) {
          float f[8], w[8];
          unpack8(xs[i], f);
          unpack8(ld_cached(wg + i), w);
#pragma unroll
          for (int j = 0; j < 8; ++j) f[j] = round_bf16(f[j] * inv) * w[j];
          xs[i] = pack8(f);
        }
      }
    } else {
      // the attention phase left (max, sum, D outputs) per head and key split: fold them
      const int D = sp.D, ns = sp.nsplit;
      for (int i = tid; i < nch; i += kStepThreads) {
        const int h = (i * 8) / D, d0 = (i * 8) - h * D;
        const int PS = D + 4;  // partial stride: D outputs, max, sum, padded to 16 bytes
        const float* src = sp.att_part + (size_t)h * ns * PS;
        float M = -INFINITY;
        for (int s = 0; s < ns; ++s) M = fmaxf(M, __ldcg(src + s * PS + D));
        float L = 0.f, acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (int s = 0; s < ns; ++s) {
          const float ms = __ldcg(src + s * PS + D);
          const float c = (ms == -INFINITY) ? 0.f : exp2f(ms - M);
          L = fmaf(__ldcg(src + s * PS + D + 1), c, L);
          const float4 o0 = __ldcg(reinterpret_cast<const float4*>(src + s * PS + d0));
          const float4 o1 = __ldcg(reinterpret_cast<const float4*>(src + s * PS + d0 + 4));
          acc[0] = fmaf(o0.x, c, acc[0]); acc[1] = fmaf(o0.y, c, acc[1]);
          acc[2] = fmaf(o0.z, c, acc[2]); acc[3] = fmaf(o0.w, c, acc[3]);
          acc[4] = fmaf(o1.x, c, acc[4]); acc[5] = fmaf(o1.y, c, acc[5]);
          acc[6] = fmaf(o1.z, c, acc[6]); acc[7] = fmaf(o1.w, c, acc[7]);
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = L > 0.f ? acc[j] / L : 0.f;
        xs[i] = pack8(acc);
      }
    }
    __syncthreads();

    for (; base < npairs; base += stride) {
      float acc0 = 0.f, acc1 = 0.f;
      const bool live_n = base + stride + g < npairs;
      int ra_n = 0, rb_n = 0;
      const uint4 *qa_n = nullptr, *qb_n = nullptr;
      if (live_n) rows_of(base + stride + g, ra_n, rb_n, qa_n, qb_n);
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
        if (lane == 0) { sh.part[warp * 2] = acc0; sh.part[warp * 2 + 1] = acc1; }
        __syncthreads();
        if (ks == 0) {
          acc0 = 0.f; acc1 = 0.f;
          for (int s = 0; s < KS; ++s) { acc0 += sh.part[(warp + s) * 2]; acc1 += sh.part[(warp + s) * 2 + 1]; }
        }
        __syncthreads();
      }
      if (live && ks == 0 && lane == 0) {
        if (MODE == PH_PLAIN) {
          float v0 = round_bf16(acc0), v1 = round_bf16(acc1);
          if (a.residual) {
            v0 = round_bf16(__fadd_rn(v0, ldcg_bf16(a.residual + ra)));
            if (rb < a.rows) v1 = round_bf16(__fadd_rn(v1, ldcg_bf16(a.residual + rb)));
          }
          a.y[ra] = __float2bfloat16_rn(v0);
          if (a.track_best) best = step_max(best, step_key(v0, ra));
          if (rb < a.rows) {
            a.y[rb] = __float2bfloat16_rn(v1);
            if (a.track_best) best = step_max(best, step_key(v1, rb));
          }
        } else if (MODE == PH_SWIGLU) {
          const float gate = round_bf16(acc0), up = round_bf16(acc1);
          const float act = round_bf16(silu_f32(gate));
          a.y[ra] = __float2bfloat16_rn(__fmul_rn(act, up));
        } else {
          const int head = ra / sp.D, i = ra - head * sp.D;
          float x1 = round_bf16(acc0), x2 = round_bf16(acc1);
          if (head < sp.H + sp.G) {
            const __nv_bfloat16* ang = sp.angles + (size_t)a.pos * sp.D;
            const float c = __bfloat162float(ang[2 * i]), s = __bfloat162float(ang[2 * i + 1]);
            const float y1 = __fsub_rn(__fmul_rn(x1, c), __fmul_rn(x2, s));
            const float y2 = __fadd_rn(__fmul_rn(x2, c), __fmul_rn(x1, s));
            x1 = y1; x2 = y2;
          }
          __nv_bfloat16* dst;
          if (head < sp.H) dst = a.y + (size_t)head * sp.D;
          else if (head < sp.H + sp.G) dst = a.k_cache + ((size_t)a.pos * sp.G + (head - sp.H)) * sp.D;
          else dst = a.v_cache + ((size_t)a.pos * sp.G + (head - sp.H - sp.G)) * sp.D;
          dst[i] = __float2bfloat16_rn(x1);
          dst[i + half] = __float2bfloat16_rn(x2);
        }
      }
      live = live_n; ra = ra_n; rb = rb_n; qa = qa_n; qb = qb_n;
    }
  }
  grid_arrive(sp.barrier);
  ++epoch;
  return true;
}

// One-query attention of every head over the cache rows [lo, pos], the keys of a head
// split over `nsplit` CTAs.  A unit is (head, split); the CTA leaves the unnormalised
// partial (D outputs, running maximum, sum) in sp.att_part for the o_proj phase to fold.
// The first batch of K and V rows is in flight before the wait for the QKV phase; the
// newest row, which that phase wrote, is read again afterwards.
template <int D>
__device__ __forceinline__ bool attention_phase(const StepParams& sp, const __nv_bfloat16* Kc,
                                                const __nv_bfloat16* Vc, int pos, StepShared& sh,
                                                float (*sm_o)[D], unsigned int& epoch) {
  constexpr int LPK = D / 8, KPW = 32 / LPK, TS = KPW * kStepWarps, UNR = 4;
  constexpr int PS = D + 4;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int dsel = lane % LPK, kslot = warp * KPW + lane / LPK;
  const int ns = sp.nsplit, units = sp.H * ns, group = sp.H / sp.G;
  const int kv_valid = pos + 1;
  const int lo = (sp.window >= 0) ? max(0, kv_valid - 1 - sp.window) : 0;
  const int per = (kv_valid - lo + ns - 1) / ns;
  const size_t row = (size_t)sp.G * D;   // elements between cache rows

  int unit = blockIdx.x;
  int h = 0, k_begin = 0, k_end = 0;
  const __nv_bfloat16 *Kb = Kc, *Vb = Vc;
  auto place = [&](int u) {
    h = u / ns;
    const int split = u - h * ns;
    k_begin = lo + split * per;
    k_end = min(kv_valid, k_begin + per);
    Kb = Kc + (size_t)(h / group) * D + dsel * 8;
    Vb = Vc + (size_t)(h / group) * D + dsel * 8;
  };
  uint4 kraw[UNR], vraw[UNR];
  auto load_batch = [&](int kb) {
#pragma unroll
    for (int u = 0; u < UNR; ++u) {
      const int k = kb + u * TS + kslot;
      const int kc = k < k_end ? k : max(k_end - 1, 0);
      kraw[u] = __ldcg(reinterpret_cast<const uint4*>(Kb + (size_t)kc * row));
      vraw[u] = __ldcg(reinterpret_cast<const uint4*>(Vb + (size_t)kc * row));
    }
  };
  bool early = false;
  if (unit < units) {
    place(unit);
    early = k_begin < k_end;
    if (early) load_batch(k_begin);
  }

  if (!grid_wait(sp.barrier, epoch, sp.status, &sh.abort)) return false;

  for (; unit < units; unit += gridDim.x) {
    if (!early) place(unit);
    float q[8], o[8], m = -INFINITY, l = 0.f;
    unpack8(__ldcg(reinterpret_cast<const uint4*>(sp.q + (size_t)h * D + dsel * 8)), q);
#pragma unroll
    for (int j = 0; j < 8; ++j) { q[j] *= sp.scale_log2; o[j] = 0.f; }
    if (early) {
#pragma unroll
      for (int u = 0; u < UNR; ++u) {
        const int k = k_begin + u * TS + kslot;
        if (k == kv_valid - 1) {
          kraw[u] = __ldcg(reinterpret_cast<const uint4*>(Kb + (size_t)k * row));
          vraw[u] = __ldcg(reinterpret_cast<const uint4*>(Vb + (size_t)k * row));
        }
      }
    }
    for (int kb = k_begin; kb < k_end; kb += TS * UNR) {
      if (!(early && kb == k_begin)) load_batch(kb);
      float s[UNR];
#pragma unroll
      for (int u = 0; u < UNR; ++u) {
        const bool live = kb + u * TS + kslot < k_end;
        float kf[8], a = 0.f;
        unpack8(kraw[u], kf);
#pragma unroll
        for (int j = 0; j < 8; ++j) a = fmaf(q[j], kf[j], a);
#pragma unroll
        for (int off = 1; off < LPK; off <<= 1) a += __shfl_xor_sync(0xffffffffu, a, off);
        s[u] = live ? a : -INFINITY;
      }
      float mn = m;
#pragma unroll
      for (int u = 0; u < UNR; ++u) mn = fmaxf(mn, s[u]);
      if (mn != -INFINITY) {
        const float corr = exp2f(m - mn);
        float pr[UNR], ps = 0.f;
#pragma unroll
        for (int u = 0; u < UNR; ++u) { pr[u] = exp2f(s[u] - mn); ps += pr[u]; }
        l = fmaf(l, corr, ps);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] *= corr;
#pragma unroll
        for (int u = 0; u < UNR; ++u) {
          float vf[8];
          unpack8(vraw[u], vf);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] = fmaf(pr[u], vf[j], o[j]);
        }
        m = mn;
      }
    }
    early = false;
    // merge the lane groups of a warp
#pragma unroll
    for (int off = LPK; off < 32; off <<= 1) {
      const float mo = __shfl_xor_sync(0xffffffffu, m, off);
      const float lo2 = __shfl_xor_sync(0xffffffffu, l, off);
      const float mn = fmaxf(m, mo);
      const float ca = (m == -INFINITY) ? 0.f : exp2f(m - mn);
      const float cb = (mo == -INFINITY) ? 0.f : exp2f(mo - mn);
      l = l * ca + lo2 * cb;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float oo = __shfl_xor_sync(0xffffffffu, o[j], off);
        o[j] = o[j] * ca + oo * cb;
      }
      m = mn;
    }
    // merge the warps into the CTA's partial
    if (lane < LPK) {
#pragma unroll
      for (int j = 0; j < 8; ++j) sm_o[warp][dsel * 8 + j] = o[j];
      if (lane == 0) { sh.att_ml[warp][0] = m; sh.att_ml[warp][1] = l; }
    }
    __syncthreads();
    float* dst = sp.att_part + (size_t)unit * PS;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < kStepWarps; ++w) M = fmaxf(M, sh.att_ml[w][0]);
    for (int d = tid; d < D + 2; d += kStepThreads) {
      float acc = 0.f;
#pragma unroll
      for (int w = 0; w < kStepWarps; ++w) {
        const float mw = sh.att_ml[w][0];
        const float c = (mw == -INFINITY) ? 0.f : exp2f(mw - M);
        acc = fmaf(d < D ? sm_o[w][d] : sh.att_ml[w][1], c, acc);
      }
      if (d < D) dst[d] = acc;
      else if (d == D) dst[D] = M;
      else dst[D + 1] = acc;
    }
    __syncthreads();
  }
  grid_arrive(sp.barrier);
  ++epoch;
  return true;
}

template <int D>
__global__ void __launch_bounds__(kStepThreads, 2) decode_step_kernel(const StepParams sp) {
  extern __shared__ uint4 xs[];
  __shared__ StepShared sh;
  __shared__ float sm_o[kStepWarps][D];
  const int tid = threadIdx.x;
  if (tid == 0) sh.abort = 0;
  __syncthreads();

  // (token, position) were left by the previous step or by the host
  int token = sp.values[0], pos = sp.values[1];
  token = max(0, min(token, sp.V - 1));
  pos = max(0, min(pos, sp.S - 1));
  unsigned int epoch = 0;
  unsigned long long best = 0ull;
  const int QD = sp.H * D, rows_qkv = (sp.H + 2 * sp.G) * D;

  for (int l = 0; l < sp.L; ++l) {
    const StepLayer& ly = sp.layers[l];
    const __nv_bfloat16* x_in = (l == 0) ? sp.embed + (size_t)token * sp.E : sp.xa;
    PhaseArgs a = {};
    a.A = ly.wqkv; a.x = x_in; a.norm_w = ly.ln1; a.y = sp.q; a.rows = rows_qkv; a.K = sp.E;
    a.plan = sp.qkv; a.stage = ST_VECTOR; a.k_cache = ly.k; a.v_cache = ly.v; a.pos = pos;
    if (!gemv_phase<PH_QKV, true>(sp, a, xs, sh, epoch, best)) return;

    if (!attention_phase<D>(sp, ly.k, ly.v, pos, sh, sm_o, epoch)) return;

    a = PhaseArgs{};
    a.A = ly.wo; a.residual = x_in; a.y = sp.xb; a.rows = sp.E; a.K = QD;
    a.plan = sp.o; a.stage = ST_ATTENTION;
    if (!gemv_phase<PH_PLAIN, true>(sp, a, xs, sh, epoch, best)) return;

    a = PhaseArgs{};
    a.A = ly.wg; a.A2 = ly.wu; a.x = sp.xb; a.norm_w = ly.ln2; a.y = sp.act; a.rows = sp.F; a.K = sp.E;
    a.plan = sp.swiglu; a.stage = ST_VECTOR;
    if (!gemv_phase<PH_SWIGLU, true>(sp, a, xs, sh, epoch, best)) return;

    a = PhaseArgs{};
    a.A = ly.wd; a.x = sp.act; a.residual = sp.xb; a.y = sp.xa; a.rows = sp.E; a.K = sp.F;
    a.plan = sp.down; a.stage = ST_VECTOR;
    if (!gemv_phase<PH_PLAIN, true>(sp, a, xs, sh, epoch, best)) return;
  }
  {
    PhaseArgs a = {};
    a.A = sp.head; a.x = sp.xa; a.norm_w = sp.final_norm; a.y = sp.logits; a.rows = sp.V; a.K = sp.E;
    a.plan = sp.headp; a.stage = ST_VECTOR; a.track_best = 1;
    // gemv_phase arrives once the CTA's rows are stored; its maximum has to be published
    // first, so the head phase is followed by one more barrier for the keys.
    if (!gemv_phase<PH_PLAIN, true>(sp, a, xs, sh, epoch, best)) return;
  }
  // ---- greedy draw: CTA maxima, then CTA 0 folds them ----
  {
    const int lane = tid & 31, warp = tid >> 5;
#pragma unroll
    for (int off = 16; off; off >>= 1) best = step_max(best, __shfl_xor_sync(0xffffffffu, best, off));
    if (lane == 0) sh.best[warp] = best;
    __syncthreads();
    if (tid == 0) {
      unsigned long long b = 0ull;
      for (int w = 0; w < kStepWarps; ++w) b = step_max(b, sh.best[w]);
      sp.best[blockIdx.x] = b;
    }
    grid_arrive(sp.barrier);
    ++epoch;
    if (blockIdx.x != 0) return;
    if (!grid_wait(sp.barrier, epoch, sp.status, &sh.abort)) return;
    unsigned long long b = 0ull;
    for (int i = tid; i < (int)gridDim.x; i += kStepThreads) b = step_max(b, __ldcg(sp.best + i));
#pragma unroll
    for (int off = 16; off; off >>= 1) b = step_max(b, __shfl_xor_sync(0xffffffffu, b, off));
    if (lane == 0) sh.best[warp] = b;
    __syncthreads();
    if (tid == 0) {
      b = 0ull;
      for (int w = 0; w < kStepWarps; ++w) b = step_max(b, sh.best[w]);
      const int drawn = (int)(~(uint32_t)(b & 0xffffffffull));
      sp.drawn[pos] = drawn;
      sp.values[0] = drawn;
      sp.values[1] = pos + 1;
    }
  }
}

// Pick the K split and the CTA count of one GEMV phase on a grid of `slots` CTAs.
static PhasePlan plan_phase(int npairs, int K, int slots) {
  const int nch = K >> 3;
  constexpr int kStep = 32 * kItem;
  int best_ks = 1;
  double best_score = -1.0;
  for (int ks = 1; ks <= kStepWarps; ks *= 2) {
    if (ks > 1 && nch / ks < kStep) break;
    const long long cta_iters = ((long long)npairs * ks + kStepWarps - 1) / kStepWarps;
    const long long waves = (cta_iters + slots - 1) / slots;
    const double eff = (double)cta_iters / (double)(waves * slots);
    const double score = cta_iters >= slots ? eff : 0.9 * (double)cta_iters / slots;
    if (score > best_score + 0.02) { best_score = score; best_ks = ks; }
  }
  const int groups = kStepWarps / best_ks;
  const long long cta_iters = (npairs + groups - 1) / groups;
  const long long waves = (cta_iters + slots - 1) / slots;
  int ctas = (int)((cta_iters + waves - 1) / waves);
  ctas = ctas < 1 ? 1 : (ctas > slots ? slots : ctas);
  return PhasePlan{best_ks, ctas};
}

template <int D>
static int launch_step(StepParams& sp, size_t smem, cudaStream_t stream) {
  static int grid = 0;
  if (grid == 0) {
    if (cudaFuncSetAttribute(decode_step_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024) !=
        cudaSuccess)
      return IRON_ERR_LAUNCH;
    int per_sm = 0, dev = 0, sms = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_step_kernel<D>, kStepThreads, 64 * 1024) !=
            cudaSuccess ||
        cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
      return IRON_ERR_LAUNCH;
    if (per_sm < 1) return IRON_ERR_LAUNCH;
    grid = (per_sm > 2 ? 2 : per_sm) * sms;
  }
  if (smem > 64 * 1024) return IRON_ERR_SHAPE;
  const int rows_qkv = (sp.H + 2 * sp.G) * sp.D;
  sp.qkv = plan_phase(rows_qkv / 2, sp.E, grid);
  sp.o = plan_phase((sp.E + 1) / 2, sp.H * sp.D, grid);
  sp.swiglu = plan_phase(sp.F, sp.E, grid);
  sp.down = plan_phase((sp.E + 1) / 2, sp.F, grid);
  sp.headp = plan_phase((sp.V + 1) / 2, sp.E, grid);
  if (cudaMemsetAsync(sp.barrier, 0, sizeof(unsigned int), stream) != cudaSuccess) return IRON_ERR_LAUNCH;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid, 1, 1);
  cfg.blockDim = dim3(kStepThreads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;   // every CTA resident: the barrier cannot starve
  attr[0].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (cudaLaunchKernelEx(&cfg, decode_step_kernel<D>, sp) != cudaSuccess) return IRON_ERR_LAUNCH;
  return IRON_OK;
}

}  // namespace iron

using namespace iron;

extern "C" size_t iron_decode_step_workspace_bytes(int H, int D) {
  // barrier word, status word, one key per CTA (at most 2 x 256 SMs), attention partials
  return 256 + 512 * sizeof(unsigned long long) + (size_t)H * 16 * (D + 4) * sizeof(float);
}

extern "C" int iron_decode_step_bf16(const void* const* layer_ptrs, int L, int E, int F, int H, int G,
                                     int D, int V, int S, const void* embed, const void* head,
                                     const void* final_norm, const void* angles, float eps,
                                     float scale, int window, int kv_len_hint, int* values,
                                     int* drawn, void* xa, void* xb, void* q, void* act, void* logits,
                                     void* workspace, iron_stream_t stream) {
  if (L <= 0 || E <= 0 || F <= 0 || H <= 0 || G <= 0 || V <= 0 || S <= 0 || H % G) return IRON_ERR_SHAPE;
  if (D != 64 && D != 128) return IRON_ERR_SHAPE;
  if ((E & 15) || (F & 15) || ((H * D) & 15)) return IRON_ERR_SHAPE;
  const void* must32[] = {embed, head, xa, xb, q, act, logits, workspace};
  for (const void* p : must32)
    if (!p || (reinterpret_cast<uintptr_t>(p) & 31u)) return IRON_ERR_ALIGN;
  if (!layer_ptrs || !final_norm || !angles || !values || !drawn) return IRON_ERR_SHAPE;
  StepParams sp = {};
  sp.layers = reinterpret_cast<const StepLayer*>(layer_ptrs);
  sp.L = L; sp.E = E; sp.F = F; sp.H = H; sp.G = G; sp.D = D; sp.V = V; sp.S = S;
  sp.embed = (const __nv_bfloat16*)embed; sp.head = (const __nv_bfloat16*)head;
  sp.final_norm = (const __nv_bfloat16*)final_norm; sp.angles = (const __nv_bfloat16*)angles;
  sp.eps = eps; sp.scale_log2 = scale * 1.4426950408889634f; sp.window = window;
  sp.values = values; sp.drawn = drawn;
  sp.xa = (__nv_bfloat16*)xa; sp.xb = (__nv_bfloat16*)xb; sp.q = (__nv_bfloat16*)q;
  sp.act = (__nv_bfloat16*)act; sp.logits = (__nv_bfloat16*)logits;
  char* ws = static_cast<char*>(workspace);
  sp.barrier = reinterpret_cast<unsigned int*>(ws);
  sp.status = reinterpret_cast<int*>(ws + 128);
  sp.best = reinterpret_cast<unsigned long long*>(ws + 256);
  sp.att_part = reinterpret_cast<float*>(ws + 256 + 512 * sizeof(unsigned long long));
  // keys of a head go to as many CTAs as the grid has per head, while each keeps a batch
  int ns = (2 * kSMs) / H;
  const int keys = kv_len_hint > 0 ? kv_len_hint : S;
  while (ns > 1 && keys / ns < 64) --ns;
  sp.nsplit = ns < 1 ? 1 : (ns > 16 ? 16 : ns);
  const int kmax = E > F ? E : F;
  const size_t smem = (size_t)(kmax > H * D ? kmax : H * D) * 2;
  return D == 64 ? launch_step<64>(sp, smem, (cudaStream_t)stream) : launch_step<128>(sp, smem, (cudaStream_t)stream);
}
