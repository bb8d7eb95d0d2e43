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

// A tensor-parallel exchange attached to a launch (iron_tp_push_next / iron_tp_pull_next).
enum { TP_NONE = 0, TP_PUSH = 1, TP_PULL = 2 };
struct TpLink {
  int mode, world, rank, slot_elems;
  unsigned char* peer[8];         // every rank's exchange buffer as this rank addresses it
  unsigned int* state;            // this rank's own: [0] the exchange's sequence number, [1] consuming CTAs done
  int* status;
  const __nv_bfloat16* residual;  // pull: added to the ranks' sum (may be null)
  __nv_bfloat16* x_out;           // pull: where CTA 0 stores the vector it built (may be null)
};

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
  int cache_rows;             // rows of the caches and of the angle table: the position is held below it
  PrefetchHint hint;          // weights a later kernel will stream (may be empty)
  TpLink tp;                  // tensor-parallel exchange this launch feeds or is fed by (mode 0: none)
};

// ---- a tensor-parallel exchange folded into the GEMVs on either side of it -----------------
// A row-parallel projection leaves every rank a partial vector that must be summed over the
// ranks and added to the residual stream before the next kernel reads it.  Instead of a
// kernel of its own, the producing GEMV stores each rounded row straight into slot
// [parity][rank] of EVERY rank's exchange buffer as one 32-bit word: the bf16 value and, in the
// upper half, a 16-bit tag of the exchange's sequence number.  A word arrives whole, so the tag
// says that its value is there: no fence and no separate flag (a system-scope fence costs
// ~5 us on this machine, more than the rest of the exchange).  The consuming GEMV, which has
// been streaming its first weights since before the producer ended, reads the slots of all
// ranks (16 bytes = four rows at a time), re-reading (bounded) any word whose tag is not yet
// this exchange's, and every CTA builds
//   x = bf16(bf16(sum over ranks, in rank order, f32) + residual)
// in shared memory where it would otherwise have staged x; CTA 0 also stores it as the next
// residual.  Slots alternate by the parity of the sequence number: a rank can be at most one
// exchange ahead of its slowest peer, so a slot is never overwritten before it is read.  The
// sequence number lives in this rank's own memory and is advanced by the last CTA of the
// consuming kernel to finish.
constexpr int kTpSlotOffset = 256;                       // bytes: the tagged slots follow the all-reduce kernel's flags
constexpr unsigned long long kTpLinkWaitNs = 2000000000ull;

__device__ __forceinline__ unsigned long long tpl_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ unsigned int tp_tag(unsigned int seq) { return ((seq >> 1) + 1u) & 0xffffu; }
__device__ __forceinline__ uint32_t* tp_slot(const TpLink& tp, int owner, unsigned int par, int rank) {
  return reinterpret_cast<uint32_t*>(tp.peer[owner] + kTpSlotOffset) + ((size_t)par * tp.world + rank) * tp.slot_elems;
}
// One rounded row value of the producing GEMV into every rank's slot.
__device__ __forceinline__ void tp_push_row(const TpLink& tp, unsigned int seq, int row, float v) {
  const uint32_t word = (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(v)) | (tp_tag(seq) << 16);
  for (int r = 0; r < tp.world; ++r)
    asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(tp_slot(tp, r, seq & 1u, tp.rank) + row), "r"(word) : "memory");
}
// The consuming side: x (n elements, n % 8 == 0) into `xs`, from the ranks' rows of the running exchange.
__device__ __forceinline__ void tp_pull_x(const TpLink& tp, uint4* xs, int n, int nthreads) {
  const int tid = threadIdx.x;
  const unsigned int seq = tp.state[0], tag = tp_tag(seq);
  const uint4* res = reinterpret_cast<const uint4*>(tp.residual);
  uint4* out = blockIdx.x == 0 && blockIdx.y == 0 ? reinterpret_cast<uint4*>(tp.x_out) : nullptr;
  unsigned long long t0 = 0;
  bool gave_up = false;
  for (int i = tid; i < (n >> 3); i += nthreads) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int r = 0; r < tp.world; ++r) {
      const uint32_t* src = tp_slot(tp, tp.rank, seq & 1u, r) + 8 * i;
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        uint32_t w0, w1, w2, w3;
        for (unsigned int it = 0;; ++it) {
          asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];"
                       : "=r"(w0), "=r"(w1), "=r"(w2), "=r"(w3) : "l"(src + 4 * h) : "memory");
          if (((w0 >> 16) == tag) & ((w1 >> 16) == tag) & ((w2 >> 16) == tag) & ((w3 >> 16) == tag)) break;
          if (gave_up) break;
          if ((it & 63u) == 63u) {
            const unsigned long long now = tpl_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > kTpLinkWaitNs) {
              gave_up = true;
              if (tp.status) *reinterpret_cast<volatile int*>(tp.status) = IRON_ERR_TIMEOUT;
              break;
            }
          }
        }
        // a word that never arrived (after the limit) counts as zero
        acc[4 * h + 0] += (w0 >> 16) == tag ? __uint_as_float(w0 << 16) : 0.f;
        acc[4 * h + 1] += (w1 >> 16) == tag ? __uint_as_float(w1 << 16) : 0.f;
        acc[4 * h + 2] += (w2 >> 16) == tag ? __uint_as_float(w2 << 16) : 0.f;
        acc[4 * h + 3] += (w3 >> 16) == tag ? __uint_as_float(w3 << 16) : 0.f;
      }
    }
    if (res) {
      float f[8];
      unpack8(ld_cached(res + i), f);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = __fadd_rn(round_bf16(acc[j]), f[j]);
    }
    const uint4 v = pack8(acc);
    xs[i] = v;
    if (out) out[i] = v;
  }
}
// The last CTA of the consuming kernel to finish moves this rank on to the next exchange.
__device__ __forceinline__ void tp_pull_done(const TpLink& tp) {
  __syncthreads();
  if (threadIdx.x != 0) return;
  const unsigned int ctas = gridDim.x * gridDim.y;
  if (atomicAdd(tp.state + 1, 1u) != ctas - 1) return;
  tp.state[1] = 0;
  tp.state[0] = tp.state[0] + 1u;
}

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;

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

  // The norm's weights do not depend on the previous kernel either: this thread's first chunk
  // of them is on its way before the wait (a second L2 round trip off the critical path).
  uint4 norm_w0 = make_uint4(0, 0, 0, 0);
  if (p.norm_mode == 2 && tid < nch) norm_w0 = ld_cached(reinterpret_cast<const uint4*>(p.norm_w) + tid);
  // The activation vector is the previous kernel's output: wait for it now.
  pdl_wait();
  const unsigned int tp_seq = p.tp.mode == TP_PUSH ? p.tp.state[0] : 0u;

  // ---- stage x (optionally RMS-normalised) into shared memory; fed by an exchange, x is
  // the ranks' sum plus the residual ----
  {
    const uint4* xg = reinterpret_cast<const uint4*>(p.x + (size_t)batch * K);
    float ss = 0.f;
    if (p.tp.mode == TP_PULL) tp_pull_x(p.tp, xs, K, kThreads);
    for (int i = tid; i < nch; i += kThreads) {
      uint4 v;
      if (p.tp.mode == TP_PULL) v = xs[i];           // written by this thread just above
      else { v = ld_cached(xg + i); xs[i] = v; }
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
          unpack8(i == tid ? norm_w0 : ld_cached(wg + i), w);
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
      if (MODE == GEMV_PLAIN && p.tp.mode == TP_PUSH) {
        tp_push_row(p.tp, tp_seq, ra, acc0);
        if (rb < p.rows) tp_push_row(p.tp, tp_seq, rb, acc1);
      } else if (MODE == GEMV_PLAIN) {
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
        const int pos = min(max(p.d_position ? *p.d_position : p.position, 0), p.cache_rows - 1);
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
  if (p.tp.mode == TP_PULL) tp_pull_done(p.tp);
}

// ---------------------------------------------------------------------------------------
// The same GEMV family with the weights streamed by the TMA engine.
//
// Two CTAs per SM, 8 warps each.  Every warp owns a ring of three 4 KB shared-memory slots; lane 0
// fills a slot with two bulk copies (cp.async.bulk + mbarrier complete_tx: 2 KB of each row
// of a pair, or 4 KB of one row) and re-arms it as soon as the warp has read it, so about
// 190 KB per SM are in flight or parked at any time without holding them in registers.  The
// first three items of every warp are issued before the programmatic-dependency wait:
// the weights do not depend on the previous kernel, so this kernel's stream starts while
// that one drains.  A pure read stream through this path runs at ~8 TB/s on a B200, above
// what register-buffered loads reach; it is used for the large matrices of a decode step
// (gate/up, down_proj, the head).  A CTA takes half an SM so that, as with the
// register-streamed kernels, the next kernel of the chain can start under this one's tail.
//   RING_PAIR   rows (2p, 2p+1)                        RING_SWIGLU  gate row m, up row m
//   RING_QKV    rows (i, i + D/2) of one head          RING_ROW     one row, 2048 columns per item
// Every mbarrier wait is bounded by a wall-clock limit; a wait that gives up leaves the
// kernel early (the rows of that warp are not written) -- there is no status word in this
// entry point's signature, so the limit is generous (2 s) and only a lost copy reaches it.
enum { RING_PAIR = 0, RING_SWIGLU = 1, RING_QKV = 2, RING_ROW = 3 };
constexpr int kRingWarps = 8;                   // two CTAs per SM, each with half of the SM's rings
constexpr int kRingCtasPerSm = 2;
constexpr int kRingThreads = kRingWarps * 32;
constexpr int kRingChunk = 1024;                 // columns of one segment
constexpr int kRingChunk16 = kRingChunk / 8;
constexpr int kRingSlotBytes = 2 * kRingChunk * 2;
constexpr int kRingSlots = 3;
constexpr int kRingMaxK = 8192;
constexpr size_t kRingBytes = (size_t)kRingWarps * kRingSlots * kRingSlotBytes;
constexpr unsigned long long kRingWaitNs = 2000000000ull;

__device__ __forceinline__ void ring_mbar_init(uint64_t* bar) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void ring_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool ring_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ void ring_bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar,
                                               uint64_t policy) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
      ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)), "l"(policy)
      : "memory");
}
__device__ __forceinline__ unsigned long long ring_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// The two segments of item `chunk` of unit `unit`: rows, first column and length of each.
template <int MODE>
__device__ __forceinline__ void ring_item(const GemvParams& p, int unit, int chunk, int& ra, int& rb,
                                          const __nv_bfloat16*& src_a, const __nv_bfloat16*& src_b, int& col_a,
                                          int& n_a, int& col_b, int& n_b) {
  const int K = p.K;
  const __nv_bfloat16* B = p.A;
  if (MODE == RING_PAIR) { ra = 2 * unit; rb = ra + 1; }
  else if (MODE == RING_SWIGLU) { ra = rb = unit; B = p.A2; }
  else if (MODE == RING_QKV) {
    const int half = p.D >> 1, head = unit / half;
    ra = head * p.D + (unit - head * half); rb = ra + half;
  } else { ra = rb = unit; }
  if (MODE == RING_ROW) {
    col_a = chunk * 2 * kRingChunk; col_b = col_a + kRingChunk;
    n_a = min(kRingChunk, K - col_a);
    n_b = max(0, min(kRingChunk, K - col_b));
  } else {
    col_a = col_b = chunk * kRingChunk;
    n_a = min(kRingChunk, K - col_a);
    n_b = (MODE == RING_PAIR && rb >= p.rows) ? 0 : n_a;
  }
  src_a = p.A + (size_t)ra * K + col_a;
  src_b = B + (size_t)(n_b ? rb : ra) * K + col_b;
}

template <int MODE>
__global__ void __launch_bounds__(kRingThreads, kRingCtasPerSm) gemv_ring_kernel(const GemvParams p, const int active_warps) {
  extern __shared__ __align__(128) unsigned char ring_smem[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int K = p.K, nch = K >> 3;
  uint4* xs = reinterpret_cast<uint4*>(ring_smem + kRingBytes);
  uint64_t* bars = reinterpret_cast<uint64_t*>(ring_smem + kRingBytes + (size_t)kRingMaxK * 2);
  float* red = reinterpret_cast<float*>(bars + kRingWarps * kRingSlots);
  if (tid == 0) {
    for (int i = 0; i < kRingWarps * kRingSlots; ++i) ring_mbar_init(bars + i);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  pdl_launch();

  // ---- this warp's units: round-robin over the active warps of the grid ----
  int units;
  if (MODE == RING_PAIR) units = (p.rows + 1) >> 1;
  else if (MODE == RING_QKV) units = p.rows >> 1;
  else units = p.rows;
  const int span = MODE == RING_ROW ? 2 * kRingChunk : kRingChunk;
  const int nchunks = (K + span - 1) / span;
  const int NW = gridDim.x * active_warps;
  const bool working = warp < active_warps;
  unsigned char* slots = ring_smem + (size_t)warp * kRingSlots * kRingSlotBytes;
  uint64_t* my_bars = bars + warp * kRingSlots;
  uint64_t policy;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));

  int i_unit = working ? warp * gridDim.x + blockIdx.x : units, i_chunk = 0, i_idx = 0;   // issue cursor
  auto issue_next = [&]() {
    if (i_unit >= units) return;
    if (lane == 0) {
      int ra, rb, col_a, n_a, col_b, n_b;
      const __nv_bfloat16 *src_a, *src_b;
      ring_item<MODE>(p, i_unit, i_chunk, ra, rb, src_a, src_b, col_a, n_a, col_b, n_b);
      const int s = i_idx % kRingSlots;
      unsigned char* dst = slots + (size_t)s * kRingSlotBytes;
      ring_expect_tx(my_bars + s, 2u * (uint32_t)(n_a + n_b));
      ring_bulk_load(dst, src_a, 2u * (uint32_t)n_a, my_bars + s, policy);
      if (n_b > 0) ring_bulk_load(dst + kRingChunk * 2, src_b, 2u * (uint32_t)n_b, my_bars + s, policy);
    }
    ++i_idx;
    if (++i_chunk == nchunks) { i_chunk = 0; i_unit += NW; }
  };
  for (int i = 0; i < kRingSlots; ++i) issue_next();

  // The norm's weights do not depend on the previous kernel either: this thread's first chunk
  // of them is on its way before the wait.
  uint4 norm_w0 = make_uint4(0, 0, 0, 0);
  if (p.norm_mode == 2 && tid < nch) norm_w0 = ld_cached(reinterpret_cast<const uint4*>(p.norm_w) + tid);
  // The activation vector is the previous kernel's output: wait for it now.
  pdl_wait();
  const unsigned int tp_seq = p.tp.mode == TP_PUSH ? p.tp.state[0] : 0u;
  {
    const uint4* xg = reinterpret_cast<const uint4*>(p.x);
    float ss = 0.f;
    if (p.tp.mode == TP_PULL) tp_pull_x(p.tp, xs, K, kRingThreads);
    for (int i = tid; i < nch; i += kRingThreads) {
      uint4 v;
      if (p.tp.mode == TP_PULL) v = xs[i];           // written by this thread just above
      else { v = ld_cached(xg + i); xs[i] = v; }
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
      for (int i = tid; i < nch; i += kRingThreads) {
        float f[8];
        unpack8(xs[i], f);
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] = round_bf16(f[j] * inv);
        if (p.norm_mode == 2) {
          float w[8];
          unpack8(i == tid ? norm_w0 : ld_cached(wg + i), w);
#pragma unroll
          for (int j = 0; j < 8; ++j) f[j] = f[j] * w[j];
        }
        xs[i] = pack8(f);
      }
    }
    __syncthreads();
  }

  float pa[4] = {0.f, 0.f, 0.f, 0.f}, pb[4] = {0.f, 0.f, 0.f, 0.f};
  int c_idx = 0;
  bool lost = false;
  for (int unit = working ? warp * gridDim.x + blockIdx.x : units; unit < units && !lost; unit += NW) {
    for (int chunk = 0; chunk < nchunks; ++chunk, ++c_idx) {
      uint64_t* bar = my_bars + c_idx % kRingSlots;
      const uint32_t parity = (uint32_t)(c_idx / kRingSlots) & 1u;
      if (!ring_try_wait(bar, parity)) {
        // The timer costs a few hundred cycles to read: the wait probes many times between
        // readings, so that a copy that lands is seen at once.
        unsigned long long t0 = 0;
        for (uint32_t it = 1; !ring_try_wait(bar, parity); ++it) {
          if ((it & 255u) != 0) continue;
          const unsigned long long now = ring_ns();
          if (t0 == 0) t0 = now;
          else if (now - t0 > kRingWaitNs) { lost = true; break; }
        }
        if (lost) break;
      }
      int ra, rb, col_a, n_a, col_b, n_b;
      const __nv_bfloat16 *src_a, *src_b;
      ring_item<MODE>(p, unit, chunk, ra, rb, src_a, src_b, col_a, n_a, col_b, n_b);
      const uint4* wa = reinterpret_cast<const uint4*>(slots + (size_t)(c_idx % kRingSlots) * kRingSlotBytes);
      const uint4* wb = wa + kRingChunk16;
      const uint4* xv = xs + (col_a >> 3);
      if (MODE == RING_ROW) {
        const int n16a = n_a >> 3, n16b = n_b >> 3;
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int i = lane + 32 * u;
          if (i < n16a) pa[u] = dot8(wa[i], xv[i], pa[u]);
          if (i < n16b) pb[u] = dot8(wb[i], xv[kRingChunk16 + i], pb[u]);
        }
      } else {
        const int n16 = n_a >> 3;
        const bool both = n_b > 0;
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int i = lane + 32 * u;
          if (i < n16) {
            const uint4 x = xv[i];
            pa[u] = dot8(wa[i], x, pa[u]);
            if (both) pb[u] = dot8(wb[i], x, pb[u]);
          }
        }
      }
      __syncwarp();     // the slot is free: start the item kRingSlots ahead
      issue_next();
      if (chunk != nchunks - 1) continue;
      float acc0 = (pa[0] + pa[1]) + (pa[2] + pa[3]);
      float acc1 = (pb[0] + pb[1]) + (pb[2] + pb[3]);
      if (MODE == RING_ROW) acc0 += acc1;
      acc0 = warp_sum(acc0);
      if (MODE != RING_ROW) acc1 = warp_sum(acc1);
#pragma unroll
      for (int u = 0; u < 4; ++u) { pa[u] = 0.f; pb[u] = 0.f; }
      if (lane != 0) continue;
      if ((MODE == RING_ROW || MODE == RING_PAIR) && p.tp.mode == TP_PUSH) {
        tp_push_row(p.tp, tp_seq, ra, acc0);
        if (MODE == RING_PAIR && rb < p.rows) tp_push_row(p.tp, tp_seq, rb, acc1);
      } else if (MODE == RING_ROW || MODE == RING_PAIR) {
        float v0 = round_bf16(acc0), v1 = round_bf16(acc1);
        if (p.residual) {
          v0 = __fadd_rn(v0, __bfloat162float(p.residual[ra]));
          if (MODE == RING_PAIR && rb < p.rows) v1 = __fadd_rn(v1, __bfloat162float(p.residual[rb]));
        }
        p.y[ra] = __float2bfloat16_rn(v0);
        if (MODE == RING_PAIR && rb < p.rows) p.y[rb] = __float2bfloat16_rn(v1);
      } else if (MODE == RING_SWIGLU) {
        const float gate = round_bf16(acc0), up = round_bf16(acc1);
        const float act = round_bf16(silu_f32(gate));
        p.y[ra] = __float2bfloat16_rn(__fmul_rn(act, up));
      } else {
        const int half = p.D >> 1;
        const int pos = min(max(p.d_position ? *p.d_position : p.position, 0), p.cache_rows - 1);
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
  }
  // copies this warp started and did not consume (only after a lost wait): let them land
  if (lost) {
    const unsigned long long t0 = ring_ns();
    for (int idx = c_idx; idx < i_idx; ++idx) {
      uint64_t* bar = my_bars + idx % kRingSlots;
      while (!ring_try_wait(bar, (uint32_t)(idx / kRingSlots) & 1u) && ring_ns() - t0 < kRingWaitNs) {}
    }
  }
  if (p.tp.mode == TP_PULL) tp_pull_done(p.tp);
}

// Which shapes go to the TMA-fed kernel (IRON_GEMV_RING, a bit mask; -1 = unset).
static int ring_policy() {
  static const int v = [] {
    const char* e = getenv("IRON_GEMV_RING");
    return e ? atoi(e) : -1;
  }();
  return v;
}

template <int MODE>
static int launch_ring(const GemvParams& p, int units, cudaStream_t stream) {
  static DeviceOnce configured;   // the attribute is per device
  constexpr size_t smem = kRingBytes + (size_t)kRingMaxK * 2 + kRingWarps * kRingSlots * 8 + 32 * sizeof(float);
  if (!configured.done()) {
    if (cudaFuncSetAttribute(gemv_ring_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
        cudaSuccess)
      return IRON_ERR_LAUNCH;
    configured.mark();
  }
  // as many warps per CTA as split the units most evenly over the grid
  int best_w = kRingWarps;
  double best_eff = -1.0;
  for (int w = kRingWarps; w >= kRingWarps / 2; --w) {
    const long long nw = (long long)kRingCtasPerSm * kSMs * w;
    const long long rounds = (units + nw - 1) / nw;
    const double eff = (double)units / (double)(rounds * nw);
    if (eff > best_eff + 1e-3) { best_eff = eff; best_w = w; }
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(kRingCtasPerSm * kSMs, 1, 1);
  cfg.blockDim = dim3(kRingThreads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  fill_pdl_attr(cfg, attr);
  if (cudaLaunchKernelEx(&cfg, gemv_ring_kernel<MODE>, p, best_w) != cudaSuccess) return IRON_ERR_LAUNCH;
  return IRON_OK;
}

template <int MODE, bool WIDE>
static int launch_gemv_w(GemvParams& p, int npairs, int batches, cudaStream_t stream) {
  static DeviceOnce configured;   // the attribute is per device
  constexpr int kMaxSmem = 100 * 1024;
  if (!configured.done()) {
    if (cudaFuncSetAttribute(gemv_kernel<MODE, WIDE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             kMaxSmem) != cudaSuccess)
      return IRON_ERR_LAUNCH;
    configured.mark();
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

// The exchange the next GEMV-family launch of this thread takes part in (consumed by it).
static thread_local TpLink g_next_link = {};
static TpLink take_tp_link() {
  TpLink l = g_next_link;
  g_next_link = TpLink{};
  return l;
}
static int set_tp_link(int mode, const void* const* h_peer_buffers, int rank, int world, int slot_elems,
                       unsigned int* d_state, int* d_status, const void* residual, void* x_out) {
  g_next_link = TpLink{};
  if (world <= 0 || world > 8 || rank < 0 || rank >= world) return IRON_ERR_SHAPE;
  if (slot_elems <= 0 || (slot_elems & 7) || !h_peer_buffers || !d_state) return IRON_ERR_SHAPE;
  if ((residual && !aligned16(residual)) || (x_out && !aligned16(x_out))) return IRON_ERR_ALIGN;
  TpLink l = {};
  l.mode = mode; l.world = world; l.rank = rank; l.slot_elems = slot_elems;
  for (int r = 0; r < world; ++r) {
    if (!h_peer_buffers[r] || !aligned16(h_peer_buffers[r])) return IRON_ERR_ALIGN;
    l.peer[r] = static_cast<unsigned char*>(const_cast<void*>(h_peer_buffers[r]));
  }
  l.state = d_state; l.status = d_status;
  l.residual = (const __nv_bfloat16*)residual; l.x_out = (__nv_bfloat16*)x_out;
  g_next_link = l;
  return IRON_OK;
}

template <int MODE>
static int launch_gemv(GemvParams& p, int npairs, int batches, cudaStream_t stream) {
  if (p.tp.mode != TP_NONE) {
    if (batches != 1 || p.repeat != 1) return IRON_ERR_UNSUPPORTED;
    if (p.tp.mode == TP_PUSH && (MODE != GEMV_PLAIN || p.residual || p.rows > p.tp.slot_elems)) return IRON_ERR_UNSUPPORTED;
    if (p.tp.mode == TP_PULL && p.K > p.tp.slot_elems) return IRON_ERR_SHAPE;
  }
  // Which shapes stream through the TMA-fed kernel: IRON_GEMV_RING is a bit mask (1 gate/up,
  // 2 large plain matrices, 4 q/k/v, 8 small plain matrices); unset = by size: gate/up always, q/k/v
  // from 24 MB, plain matrices from 16 MB.  Measured on the Llama-3.2-1B decode step: gate/up 12.3 us
  // against 14.5 us register-streamed; the whole step 695 us with mask 3, 710 us with 0, 704 us with
  // 15 (its 12.6 MB q/k/v matrix gains nothing); on the 3B step (31.5 MB q/k/v, 18.9 MB o_proj)
  // 1.686 ms with mask 3, 1.651 with 7, 1.648 with 15.
  const int policy = ring_policy();
  const long long bytes = (long long)p.rows * p.K * 2 * (MODE == GEMV_SWIGLU ? 2 : 1);
  const int by_size = 1 | (bytes >= (24ll << 20) ? 4 : 0) | (bytes >= (16ll << 20) ? 2 | 8 : 0);
  const int mask = policy >= 0 ? policy : by_size;
  if (mask && batches == 1 && p.repeat == 1 && p.K <= kRingMaxK) {
    if (MODE == GEMV_SWIGLU && (mask & 1)) return launch_ring<RING_SWIGLU>(p, p.rows, stream);
    if (MODE == GEMV_QKV && (mask & 4)) return launch_ring<RING_QKV>(p, p.rows >> 1, stream);
    if (MODE == GEMV_PLAIN && (mask & (bytes >= (24ll << 20) ? 2 : 8))) {
      if (npairs < kRingCtasPerSm * kSMs * kRingWarps) return launch_ring<RING_ROW>(p, p.rows, stream);
      return launch_ring<RING_PAIR>(p, npairs, stream);
    }
  }
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
  const TpLink link = take_tp_link();   // consumed by this call whatever it returns
  int rc = check_common(A, x, y, M, K);
  if (rc) return rc;
  if (batches <= 0 || repeat <= 0 || batches % repeat) return IRON_ERR_SHAPE;
  if (valid_rows < 0 || valid_rows > M) return IRON_ERR_SHAPE;
  if (norm_mode < 0 || norm_mode > 2 || (norm_mode == 2 && !norm_weight)) return IRON_ERR_SHAPE;
  if (norm_mode == 2 && !aligned16(norm_weight)) return IRON_ERR_ALIGN;
  if (valid_rows == 0) return link.mode == TP_NONE ? IRON_OK : IRON_ERR_UNSUPPORTED;
  GemvParams p = {};
  p.tp = link;
  p.A = (const __nv_bfloat16*)A; p.x = (const __nv_bfloat16*)x; p.y = (__nv_bfloat16*)y;
  p.residual = (const __nv_bfloat16*)residual; p.norm_w = (const __nv_bfloat16*)norm_weight;
  p.M = M; p.K = K; p.repeat = repeat; p.rows = valid_rows; p.norm_mode = norm_mode; p.eps = eps;
  return launch_gemv<GEMV_PLAIN>(p, (valid_rows + 1) / 2, batches, (cudaStream_t)stream);
}

extern "C" int iron_tp_push_next(const void* const* h_peer_buffers, int rank, int world, int slot_elems,
                                 unsigned int* d_state, int* d_status) {
  return set_tp_link(TP_PUSH, h_peer_buffers, rank, world, slot_elems, d_state, d_status, nullptr, nullptr);
}

extern "C" int iron_tp_pull_next(const void* const* h_peer_buffers, int rank, int world, int slot_elems,
                                 unsigned int* d_state, int* d_status, const void* residual, void* x_out) {
  return set_tp_link(TP_PULL, h_peer_buffers, rank, world, slot_elems, d_state, d_status, residual, x_out);
}

extern "C" int iron_gemv_swiglu_bf16(const void* Wg, const void* Wu, const void* x, void* y,
                                     int M, int K, int norm_mode, const void* norm_weight,
                                     float eps, iron_stream_t stream) {
  const TpLink link = take_tp_link();
  int rc = check_common(Wg, x, y, M, K);
  if (rc) return rc;
  if (!aligned16(Wu)) return IRON_ERR_ALIGN;
  if (norm_mode < 0 || norm_mode > 2 || (norm_mode == 2 && !norm_weight)) return IRON_ERR_SHAPE;
  GemvParams p = {};
  p.tp = link;
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
                                         int cache_rows, iron_stream_t stream) {
  const TpLink link = take_tp_link();
  if (H <= 0 || G <= 0 || D <= 0 || (D & 15) || cache_rows <= 0) return IRON_ERR_SHAPE;
  const int M = (H + 2 * G) * D;
  int rc = check_common(Wqkv, x, q_out, M, K);
  if (rc) return rc;
  if (!angles || !k_cache || !v_cache) return IRON_ERR_SHAPE;
  if (norm_mode < 0 || norm_mode > 2 || (norm_mode == 2 && !norm_weight)) return IRON_ERR_SHAPE;
  if (!d_position && (position < 0 || position >= cache_rows)) return IRON_ERR_SHAPE;
  GemvParams p = {};
  p.tp = link;
  p.A = (const __nv_bfloat16*)Wqkv; p.x = (const __nv_bfloat16*)x; p.y = (__nv_bfloat16*)q_out;
  p.norm_w = (const __nv_bfloat16*)norm_weight;
  p.M = M; p.K = K; p.repeat = 1; p.rows = M; p.norm_mode = norm_mode; p.eps = eps;
  p.angles = (const __nv_bfloat16*)angles;
  p.k_cache = (__nv_bfloat16*)k_cache; p.v_cache = (__nv_bfloat16*)v_cache;
  p.d_position = d_position; p.position = position; p.H = H; p.G = G; p.D = D;
  p.cache_rows = cache_rows;
  return launch_gemv<GEMV_QKV>(p, M / 2, 1, (cudaStream_t)stream);
}
