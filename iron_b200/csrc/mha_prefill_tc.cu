// Prompt-chunk attention on the 5th-generation tensor cores.
//
// One CTA = 128 query rows of one head; keys and values stream in 128-row tiles:
//   warp 0      TMA producer: the Q tile once, then K and V tiles into two rings
//               (4-D tensor maps over (d, head, row, batch), 128-byte swizzle)
//   warp 1      issues S = Q K^T (M 128, N 128, K = D) into one of two 128-column
//               accumulators in tensor memory, as far ahead as they and the K ring allow
//   warp 10     issues PV = P V (M 128, N = D, K = 128 keys, V read N-major as it lies in
//               the cache) into one of two D-column accumulators as each P arrives; an
//               issuing thread spends ~100 cycles per instruction, so one thread for both
//               products made the issue, not the tensor pipe, the limit
//   warps 2..9  softmax: two threads own one query row (one TMEM lane), each half of the
//               tile's keys and half of the output row, so a sub-partition has two warps
//               to hide each other's latencies.  A thread reads its 64 scores once (and the
//               other half's for the row maximum, so the two agree on it without meeting), writes P as bf16 into shared
//               memory in the operand layout the second MMA reads, and keeps its half of
//               the output row in registers: o = o * exp2(m_old - m_new) + PV.
// S of tile i+1 is issued before PV of tile i, so the tensor core works on the next scores
// while the softmax of the current tile runs; the exponentials (one per score, on the
// special-function unit) are what bounds the kernel.
// CTAs are persistent (one per SM): each walks its share of the (query block, head, sequence)
// items, long key ranges first, so tensor memory and the barriers are set up once and the
// next item's tiles load under the current item's last ones.
//
// The arithmetic is the warp-MMA kernel's: scores scaled in the exp2 domain, P rounded to
// bf16 for the second product, the row sum taken over the unrounded exponentials, one
// division at the end; masking by position (causal and/or window) and by the key bound.
// Every mbarrier wait is bounded; a wait that gives up sets the abort flag, every role
// unwinds, tensor memory is freed and the status word receives IRON_ERR_TIMEOUT.
#include <cstdio>
#include <cstdlib>

#include "common.cuh"
#include "tc.cuh"

namespace iron {

struct PrefillTcParams {
  __nv_bfloat16* O;
  long long o_batch_stride, o_row_stride, o_head_stride;
  int H, G, batch, q_rows, q_tokens, kv_tokens, causal, window;
  float scale_log2;
  int* status;
  long long* trace;
};

constexpr int kTcThreads = 352;   // producer, S issuer, eight softmax warps, PV issuer
constexpr int kTcM = 128;      // query rows of a CTA
constexpr int kTcN = 128;      // keys of a tile
constexpr uint32_t kMmaHintNs = 64;   // the producer and the MMA issuer sleep in short naps: a late wake-up delays the pipeline
constexpr int kSub = 16384;    // one 128-row x 64-element (128-byte, swizzled) sub-tile

template <int D>
struct TcCfg {
  static constexpr int kChunks = D / 64;                    // sub-tiles of a Q, K or V tile
  static constexpr int kTile = kChunks * kSub;
  static constexpr int kStages = D == 64 ? 3 : 2;
  static constexpr int kQ = 0;
  static constexpr int kK = kQ + kTile;
  static constexpr int kV = kK + kStages * kTile;
  static constexpr int kP = kV + kStages * kTile;           // 2 buffers x 2 sub-tiles (keys 0..63, 64..127)
  static constexpr int kBars = kP + 2 * 2 * kSub;
  static constexpr int kXch = kBars + 256;                  // the halves' row sums meet here
#ifdef TC_TRACE
  static constexpr int kSmem = kXch + 2 * kTcM * 4 + 64 + 1024;
#else
  static constexpr int kSmem = kXch + 2 * kTcM * 4 + 1024;
#endif
  static constexpr int kColsS = 0;                          // 2 x 128 columns
  static constexpr int kColsPV = 256;                       // 2 x D columns
};

__device__ __forceinline__ void tma_load_4d(void* dst, const CUtensorMap* map, int x, int h, int row, int b,
                                            uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(x), "r"(h), "r"(row), "r"(b), "r"(smem_u32(bar))
      : "memory");
}
// Two non-negative floats rounded to bf16 (to nearest, ties away from zero) and packed, on the
// integer pipes: the conversion instruction shares the special-function unit with the
// exponentials, which is the unit this kernel is bound by.
__device__ __forceinline__ uint32_t pack_bf16x2_alu(float lo, float hi) {
  const uint32_t a = __float_as_uint(lo) + 0x8000u, b = __float_as_uint(hi) + 0x8000u;
  return __byte_perm(a, b, 0x7632);
}
__device__ __forceinline__ float ex2_ftz(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// kind::f16 instruction descriptor: bf16 x bf16 -> f32, M 128, A K-major.
__host__ __device__ constexpr uint32_t tc_idesc(int n, bool b_n_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((b_n_major ? 1u : 0u) << 16) | ((uint32_t)(n >> 3) << 17) |
         ((uint32_t)(kTcM >> 4) << 24);
}

// What a CTA works on: 128 query rows of one head of one sequence, and the key tiles they see.
struct TcItem {
  int b, head, kvh, m0, j_lo, n_tiles;
};

template <int D>
__global__ void __launch_bounds__(kTcThreads, 1)
mha_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                      const __grid_constant__ CUtensorMap map_v, const PrefillTcParams p) {
  using Cfg = TcCfg<D>;
  extern __shared__ uint8_t tc_smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(tc_smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::kBars);
  uint64_t* q_full = bars;                       // [1]
  uint64_t* q_empty = bars + 1;                  // [1]
  uint64_t* k_full = bars + 2;                   // [kStages]
  uint64_t* k_empty = k_full + Cfg::kStages;
  uint64_t* v_full = k_empty + Cfg::kStages;
  uint64_t* v_empty = v_full + Cfg::kStages;
  uint64_t* s_full = v_empty + Cfg::kStages;     // [2]
  uint64_t* s_empty = s_full + 2;
  uint64_t* p_full = s_empty + 2;
  uint64_t* pv_full = p_full + 2;                // PV done: the result is ready and the P buffer is free
  uint64_t* pv_empty = pv_full + 2;
  uint64_t* x_bar = pv_empty + 2;                // [1] the two halves of a row meet here
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(x_bar + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* xch = reinterpret_cast<float*>(smem + Cfg::kXch);   // [2 halves][128 rows]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q_tokens = p.q_tokens, kv_tokens = p.kv_tokens;
  const bool masked = p.causal || p.window >= 0;
  const int offset = masked ? kv_tokens - q_tokens : 0;   // position of query row 0 (>= 0: checked on the host)

  // The CTAs are persistent: item w of the launch is query block (late blocks, the long key
  // ranges, first) x head (fastest) x sequence; CTA c takes items c, c + grid, ... so every
  // CTA gets a long item, then shorter ones, and the next item's tiles load (and its first
  // scores are computed) under the current item's tail.
  const int q_blocks = (q_tokens + kTcM - 1) / kTcM;
  const int per_seq = q_blocks * p.H;
  const int total = per_seq * p.batch;
  // The k-th item of this CTA: rounds of gridDim.x items, walked forwards and backwards in
  // turn, so a CTA that got the longest item of one round gets the shortest of the next.
  // Returns `total` when the CTA has no k-th item.
  auto work = [&](int k) {
    const int base = k * (int)gridDim.x;
    if (base >= total) return total;
    const int w = base + ((k & 1) ? (int)gridDim.x - 1 - (int)blockIdx.x : (int)blockIdx.x);
    return w < total ? w : total;
  };
  auto item_of = [&](int w) {
    TcItem it;
    it.b = w / per_seq;
    const int rem = w - it.b * per_seq;
    it.head = rem % p.H;
    it.kvh = it.head / (p.H / p.G);
    it.m0 = (q_blocks - 1 - rem / p.H) * kTcM;
    int j_lo = 0, j_hi = (kv_tokens + kTcN - 1) / kTcN;
    const int last_row = min(it.m0 + kTcM, q_tokens) - 1;
    if (p.causal) j_hi = min(j_hi, (offset + last_row) / kTcN + 1);
    else if (p.window >= 0) j_hi = min(j_hi, (offset + last_row + p.window) / kTcN + 1);
    if (p.window >= 0) j_lo = max(0, (offset + it.m0 - p.window) / kTcN);
    it.j_lo = j_lo;
    it.n_tiles = j_hi - j_lo;   // >= 1: the block has a live row and that row sees its own key
    return it;
  };

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    mbar_init(q_empty, 1);
    for (int s = 0; s < Cfg::kStages; ++s) {
      mbar_init(k_full + s, 1); mbar_init(k_empty + s, 1); mbar_init(v_full + s, 1); mbar_init(v_empty + s, 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(s_full + a, 1); mbar_init(s_empty + a, 256);
      mbar_init(p_full + a, 256);
      mbar_init(pv_full + a, 1); mbar_init(pv_empty + a, 256);
    }
    mbar_init(x_bar, 256);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_q) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_k) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_v) : "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"(512)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  pdl_launch();
  pdl_wait();   // Q, K and V are the previous kernels' outputs

  if (warp == 0) {
    // ---------------- producer ----------------
    if (lane == 0) {
      int s = 0, issued = 0, n_item = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int w = work(0); w < total && ok; w = work(++n_item)) {
        const TcItem it = item_of(w);
        // the Q tile is single: the previous item's last S product must have read it
        if (!mbar_wait_relaxed(q_empty, (n_item & 1) ^ 1, abort_flag, kMmaHintNs)) { ok = false; break; }
        mbar_expect_tx(q_full, Cfg::kTile);
#pragma unroll
        for (int c = 0; c < Cfg::kChunks; ++c)
          tma_load_4d(smem + Cfg::kQ + c * kSub, &map_q, c * 64, it.head, it.m0, it.b, q_full);
        ++issued;
        for (int i = 0; i < it.n_tiles && ok; ++i) {
          const int row = (it.j_lo + i) * kTcN;
          if (!mbar_wait_relaxed(k_empty + s, phase ^ 1, abort_flag, kMmaHintNs)) { ok = false; break; }
          mbar_expect_tx(k_full + s, Cfg::kTile);
#pragma unroll
          for (int c = 0; c < Cfg::kChunks; ++c)
            tma_load_4d(smem + Cfg::kK + s * Cfg::kTile + c * kSub, &map_k, c * 64, it.kvh, row, it.b, k_full + s);
          if (!mbar_wait_relaxed(v_empty + s, phase ^ 1, abort_flag, kMmaHintNs)) { ok = false; break; }
          mbar_expect_tx(v_full + s, Cfg::kTile);
#pragma unroll
          for (int c = 0; c < Cfg::kChunks; ++c)
            tma_load_4d(smem + Cfg::kV + s * Cfg::kTile + c * kSub, &map_v, c * 64, it.kvh, row, it.b, v_full + s);
          if (++s == Cfg::kStages) { s = 0; phase ^= 1; }
        }
      }
      if (!ok && issued > 0) {
        // Unwinding: give the copies in flight a millisecond, many times what one takes.
        const unsigned long long t0 = global_ns();
        while (global_ns() - t0 < 1000000ull) {}
      }
    }
  } else if (warp == 1 || warp == 10) {
    // ---------------- MMA issuers ----------------
    if (lane == 0) {
      constexpr uint32_t idesc_s = tc_idesc(kTcN, false);
      constexpr uint32_t idesc_pv = tc_idesc(D, true);
      // Descriptors are built once; a K step or a stage only moves the 14-bit address field
      // (16-byte units), which the issuing thread adds: it runs alone, so every instruction
      // it spends between two MMAs is exposed.
      const uint64_t q_desc = make_desc(smem_u32(smem + Cfg::kQ), 16, 1024);
      const uint64_t k_desc0 = make_desc(smem_u32(smem + Cfg::kK), 16, 1024);
      const uint64_t p_desc0 = make_desc(smem_u32(smem + Cfg::kP), 16, 1024);
      const uint64_t v_desc0 = make_desc(smem_u32(smem + Cfg::kV), kSub, 1024);
      auto issue_s = [&](int stage, int sb) {
        const uint64_t k_desc = k_desc0 + (uint64_t)((stage * Cfg::kTile) >> 4);
        const uint32_t d_tmem = tmem_base + Cfg::kColsS + sb * kTcN;
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
#ifdef TC_SKIP_S
          if (k > 0) break;
#endif
          constexpr int kStep = 32 >> 4, kSubStep = kSub >> 4;   // 32 bytes per K step within a 64-element sub-tile
          const uint64_t off = (uint64_t)((k >> 2) * kSubStep + (k & 3) * kStep);
          tcgen05_mma_bf16(d_tmem, q_desc + off, k_desc + off, idesc_s, k != 0);
        }
      };
      auto issue_pv = [&](int stage, int pb) {
        const uint64_t v_desc = v_desc0 + (uint64_t)((stage * Cfg::kTile) >> 4);
        const uint64_t p_desc = p_desc0 + (uint64_t)((pb * 2 * kSub) >> 4);
        const uint32_t d_tmem = tmem_base + Cfg::kColsPV + pb * D;
#pragma unroll
        for (int k = 0; k < kTcN / 16; ++k) {
#ifdef TC_SKIP_PV
          if (k > 0) break;
#endif
          // A = P, K-major: key sub-tile k / 4, 32 bytes per step.  B = V, N-major: 16 key
          // rows of 128 bytes per step, 64-element column chunks one sub-tile apart.
          tcgen05_mma_bf16(d_tmem, p_desc + (uint64_t)((k >> 2) * (kSub >> 4) + (k & 3) * 2),
                           v_desc + (uint64_t)((k * 16 * 128) >> 4), idesc_pv, k != 0);
        }
      };
#ifdef TC_TRACE
      long long mt[6] = {0, 0, 0, 0, 0, 0};
      long long mc0 = clock64();
#define MMA_MARK(k) { const long long now = clock64(); mt[k] += now - mc0; mc0 = now; }
#else
#define MMA_MARK(k)
#endif
      // Two issuers, so that neither product waits for the other's instructions to be issued:
      // warp 1 issues S for every tile of every item in turn, as far ahead as the two S
      // accumulators and the K ring allow; warp 10 issues PV as each P arrives.  Tiles are
      // counted over the whole launch (`t`): t & 1 picks the accumulator, t >> 1 its phase.
      int stage = 0, t = 0, n_item = 0;
      uint32_t phase = 0;
      bool ok = true;
      if (warp == 1) {
        for (int w = work(0); w < total && ok; w = work(++n_item)) {
          const TcItem it = item_of(w);
          if (!mbar_wait_relaxed(q_full, n_item & 1, abort_flag, kMmaHintNs)) { ok = false; break; }
          for (int i = 0; i < it.n_tiles; ++i, ++t) {
            const int sb = t & 1;
            MMA_MARK(5)
            if (!mbar_wait_relaxed(k_full + stage, phase, abort_flag, kMmaHintNs)) { ok = false; break; }
            MMA_MARK(0)
            if (!mbar_wait_relaxed(s_empty + sb, ((t >> 1) & 1) ^ 1, abort_flag, kMmaHintNs)) { ok = false; break; }
            MMA_MARK(1)
            tcgen05_fence_after();
#ifdef TC_TRACE
            reinterpret_cast<volatile long long*>(smem + Cfg::kXch + 1024)[t & 7] = clock64();
#endif
            issue_s(stage, sb);
            tcgen05_commit(k_empty + stage);
            if (i + 1 == it.n_tiles) tcgen05_commit(q_empty);   // the Q tile is free for the next item
            tcgen05_commit(s_full + sb);
            if (++stage == Cfg::kStages) { stage = 0; phase ^= 1; }
          }
        }
      } else {
        for (int w = work(0); w < total && ok; w = work(++n_item)) {
          const TcItem it = item_of(w);
          for (int i = 0; i < it.n_tiles; ++i, ++t) {
            const int pb = t & 1;
            const uint32_t ph = (t >> 1) & 1;
            MMA_MARK(5)
            if (!mbar_wait_relaxed(v_full + stage, phase, abort_flag, kMmaHintNs)) { ok = false; break; }
            MMA_MARK(2)
            if (!mbar_wait_relaxed(p_full + pb, ph, abort_flag, kMmaHintNs)) { ok = false; break; }
            MMA_MARK(3)
            if (!mbar_wait_relaxed(pv_empty + pb, ph ^ 1, abort_flag, kMmaHintNs)) { ok = false; break; }
            MMA_MARK(4)
            tcgen05_fence_after();
            issue_pv(stage, pb);
            tcgen05_commit(v_empty + stage);
            tcgen05_commit(pv_full + pb);
            if (++stage == Cfg::kStages) { stage = 0; phase ^= 1; }
          }
        }
      }
#ifdef TC_TRACE
      if (p.trace && blockIdx.x < 8) {
        const int base = 64 + (warp == 1 ? 0 : 64) + blockIdx.x * 8;
        for (int k = 0; k < 6; ++k) p.trace[base + k] = mt[k];
        p.trace[base + 6] = t;
      }
#endif
    }
  } else if (warp < 10) {
    // ---------------- softmax and output (warps 2..9) ----------------
    // Two threads share a query row: warps 2..5 take keys 0..63 of each tile and the first
    // half of the output row, warps 6..9 keys 64..127 and the second half.  Their row sums
    // meet once per item, at its end, in shared memory under a bounded mbarrier.
    const int quarter = warp & 3;             // the TMEM lanes this warp may read
    const int half = (warp - 2) >> 2;
    const int r = quarter * 32 + lane;        // row of the tile
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
    constexpr int DH = D / 2;                 // output columns of this thread
    constexpr int KH = kTcN / 2;              // keys of a tile of this thread
    const float scale = p.scale_log2;         // > 0: the maximum commutes with the scaling
    bool ok = true;
    int g = 0, n_item = 0;
#ifdef TC_TRACE
    long long tr[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    long long tc0 = clock64();
#define TC_MARK(k) { const long long now = clock64(); tr[k] += now - tc0; tc0 = now; }
#else
#define TC_MARK(k)
#endif

    for (int w = work(0); w < total && ok; w = work(++n_item)) {
      const TcItem it = item_of(w);
      const int row = it.m0 + r;
      const int pos = offset + row;           // position of this query
      float o[DH];
#pragma unroll
      for (int d = 0; d < DH; ++d) o[d] = 0.f;
      float m_run = -INFINITY, l_run = 0.f, corr_prev = 0.f;

      // o = o * corr + PV of tile `t` (corr: that tile's rescale), then the PV buffer is free
      auto add_pv = [&](int t, float corr) -> bool {
        const int pb = t & 1;
        if (!mbar_wait(pv_full + pb, (t >> 1) & 1, abort_flag)) return false;
        tcgen05_fence_after();
        uint32_t v[DH];
#pragma unroll
        for (int c = 0; c < DH / 32; ++c) tmem_ld32(lane_addr + Cfg::kColsPV + pb * D + half * DH + c * 32, v + c * 32);
        tmem_ld_wait();
        tcgen05_fence_before();
        mbar_arrive(pv_empty + pb);
#pragma unroll
        for (int j = 0; j < DH; ++j) o[j] = fmaf(o[j], corr, __uint_as_float(v[j]));
        return true;
      };
      auto key_live = [&](int key) {
        bool k_ok = key < kv_tokens;
        if (p.causal) k_ok = k_ok && key <= pos;
        else if (p.window >= 0) k_ok = k_ok && key <= pos + p.window;
        if (p.window >= 0) k_ok = k_ok && key >= pos - p.window;
        return k_ok;
      };

      for (int i = 0; i < it.n_tiles && ok; ++i) {
        const int t = g + i, sb = t & 1;
        const uint32_t ph = (t >> 1) & 1;
        const int tile0 = (it.j_lo + i) * kTcN, key0 = tile0 + half * KH;
        const bool partial =
            (tile0 + kTcN > kv_tokens) || p.window >= 0 || (p.causal && tile0 + kTcN - 1 > offset + it.m0);
#ifdef TC_TRACE
        const bool first_try = mbar_try_wait(s_full + sb, ph);
        const long long t_before = clock64();
#endif
        if (!mbar_wait(s_full + sb, ph, abort_flag)) { ok = false; break; }
#ifdef TC_TRACE
        {
          const long long now = clock64();
          tr[7] += first_try ? 1 : 0;
          tr[6] += now - reinterpret_cast<volatile long long*>(smem + Cfg::kXch + 1024)[t & 7];   // issue -> observed
          (void)t_before;
        }
#endif
        tcgen05_fence_after();
        TC_MARK(0)
        // this thread's 64 scores stay in registers; the other half's are read for the maximum
        // only, so the two threads of a row agree on it without meeting
        uint32_t sc[KH];
        float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
        const uint32_t s_addr = lane_addr + Cfg::kColsS + sb * kTcN;
#pragma unroll
        for (int c = 0; c < KH / 32; ++c) tmem_ld32(s_addr + half * KH + c * 32, sc + c * 32);
#pragma unroll
        for (int c = 0; c < KH / 32; ++c) {
          uint32_t so[32];
          tmem_ld32(s_addr + (half ^ 1) * KH + c * 32, so);
          tmem_ld_wait();
          if (c == KH / 32 - 1) {   // every score needed is in registers: the accumulator may be overwritten
            tcgen05_fence_before();
            mbar_arrive(s_empty + sb);
          }
          if (partial) {
            const int other0 = tile0 + (half ^ 1) * KH + c * 32;
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (!key_live(other0 + j)) so[j] = 0xff800000u;   // -inf
          }
#pragma unroll
          for (int j = 0; j < 32; ++j) mx4[j & 3] = fmaxf(mx4[j & 3], __uint_as_float(so[j]));
        }
        if (partial) {
#pragma unroll
          for (int j = 0; j < KH; ++j)
            if (!key_live(key0 + j)) sc[j] = 0xff800000u;
        }
#pragma unroll
        for (int j = 0; j < KH; ++j) mx4[j & 3] = fmaxf(mx4[j & 3], __uint_as_float(sc[j]));
        const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * scale;
        const float m_new = fmaxf(m_run, mx);
        const float msafe = (m_new == -INFINITY) ? 0.f : m_new;
        const float corr = ex2_ftz(m_run - msafe);   // m_run = -inf gives 0
        m_run = m_new;
        TC_MARK(1)
        // the P buffer is free once the PV product two tiles back has read it
        if (!mbar_wait(pv_full + sb, ph ^ 1, abort_flag)) { ok = false; break; }
        TC_MARK(2)
        // exponentials, their sum, and P in the MMA's operand layout: this thread's 64 keys
        // are one 128-byte row of sub-tile `half`
        uint8_t* p_row = smem + Cfg::kP + sb * 2 * kSub + half * kSub + r * 128;
        float ls4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int g8 = 0; g8 < KH / 8; ++g8) {
          uint32_t packed[4];
#pragma unroll
          for (int j = 0; j < 8; j += 2) {
            const float p0 = ex2_ftz(fmaf(__uint_as_float(sc[g8 * 8 + j]), scale, -msafe));
            const float p1 = ex2_ftz(fmaf(__uint_as_float(sc[g8 * 8 + j + 1]), scale, -msafe));
            ls4[(j >> 1) & 3] += p0 + p1;
            packed[j >> 1] = pack_bf16x2_alu(p0, p1);
          }
          *reinterpret_cast<uint4*>(p_row + ((g8 ^ (r & 7)) << 4)) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
        }
        TC_MARK(5)
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        mbar_arrive(p_full + sb);
        TC_MARK(3)
        l_run = l_run * corr + ((ls4[0] + ls4[1]) + (ls4[2] + ls4[3]));
        // the previous tile's PV joins the row, rescaled by that tile's factor
        if (i > 0 && !add_pv(t - 1, corr_prev)) { ok = false; break; }
        corr_prev = corr;
        TC_MARK(4)
      }
      if (ok) ok = add_pv(g + it.n_tiles - 1, corr_prev);
      // the halves' row sums meet, under a bounded wait
      float l_other = 0.f;
      if (ok) {
        xch[half * kTcM + r] = l_run;
        mbar_arrive(x_bar);
        ok = mbar_wait(x_bar, n_item & 1, abort_flag);
        if (ok) l_other = xch[(half ^ 1) * kTcM + r];
      }
      if (ok && row < p.q_rows) {
        const float l = half == 0 ? l_run + l_other : l_other + l_run;   // one order for both threads
        const float inv = (row < q_tokens && l > 0.f) ? 1.0f / l : 0.f;
        __nv_bfloat16* dst = p.O + (long long)it.b * p.o_batch_stride + (long long)it.head * p.o_head_stride +
                             (long long)row * p.o_row_stride + half * DH;
#pragma unroll
        for (int c = 0; c < DH / 8; ++c) {
          float f[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) f[j] = o[c * 8 + j] * inv;
          *reinterpret_cast<uint4*>(dst + c * 8) = pack8(f);
        }
      }
      g += it.n_tiles;
    }
#ifdef TC_TRACE
    if (p.trace && r == 0 && half == 0 && blockIdx.x < 8) {
      for (int k = 0; k < 7; ++k) p.trace[blockIdx.x * 8 + k] = tr[k];
      p.trace[blockIdx.x * 8 + 7] = g * 1000 + tr[7];
    }
#endif
    // rows between the query bound's last block and the end of the buffer are zeros
    const int z0 = q_blocks * kTcM;
    if (z0 < p.q_rows) {
      const int zrows = p.q_rows - z0, per_row = D / 8;
      const long long cells = (long long)p.batch * p.H * zrows * per_row;
      for (long long idx = (long long)blockIdx.x * 256 + (threadIdx.x - 64); idx < cells; idx += (long long)gridDim.x * 256) {
        const int c = (int)(idx % per_row);
        const int zr = (int)((idx / per_row) % zrows);
        const int hh = (int)((idx / ((long long)per_row * zrows)) % p.H);
        const int bb = (int)(idx / ((long long)per_row * zrows * p.H));
        *reinterpret_cast<uint4*>(p.O + (long long)bb * p.o_batch_stride + (long long)hh * p.o_head_stride +
                                  (long long)(z0 + zr) * p.o_row_stride + c * 8) = make_uint4(0, 0, 0, 0);
      }
    }
  }

  tcgen05_fence_before();
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag && p.status) *p.status = IRON_ERR_TIMEOUT;
  if (warp == 1) {
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
  }
}

// ---- host side ---------------------------------------------------------------
#ifdef TC_TRACE
long long* g_tc_trace = nullptr;
#endif
typedef CUresult (*TcEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                               const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                               CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static TcEncodeFn tc_encode() {
  static TcEncodeFn fn = nullptr;
  if (!fn) {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<TcEncodeFn>(sym);
  }
  return fn;
}

// (d, head, row, batch) over a bf16 tensor with element strides; boxes of 64 x 1 x 128 x 1.
static bool tc_map(CUtensorMap* map, const void* base, int D, int heads, int rows, int batch, long long head_stride,
                   long long row_stride, long long batch_stride) {
  TcEncodeFn fn = tc_encode();
  if (!fn || rows <= 0) return false;
  if (batch == 1) batch_stride = row_stride * rows;   // unused, but must be a valid stride
  const cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)heads, (cuuint64_t)rows, (cuuint64_t)batch};
  const cuuint64_t strides[3] = {(cuuint64_t)head_stride * 2, (cuuint64_t)row_stride * 2,
                                 (cuuint64_t)batch_stride * 2};
  const cuuint32_t box[4] = {64, 1, (cuuint32_t)kTcN, 1};
  const cuuint32_t elem[4] = {1, 1, 1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, elem,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int D>
static int launch_prefill_tc(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv,
                             const PrefillTcParams& p, int batch, cudaStream_t stream) {
  using Cfg = TcCfg<D>;
  static DeviceOnce configured;   // the attribute is per device
  if (!configured.done()) {
    const cudaError_t e =
        cudaFuncSetAttribute(mha_prefill_tc_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmem);
    if (e != cudaSuccess) {
      if (getenv("IRON_DEBUG")) fprintf(stderr, "mha_prefill_tc<%d> smem %d: %s\n", D, Cfg::kSmem, cudaGetErrorString(e));
      return IRON_ERR_LAUNCH;
    }
    configured.mark();
  }
  cudaLaunchConfig_t cfg = {};
  const int items = ((p.q_tokens + kTcM - 1) / kTcM) * p.H * batch;
  cfg.gridDim = dim3(items < kSMs ? items : kSMs);
  cfg.blockDim = dim3(kTcThreads);
  cfg.dynamicSmemBytes = Cfg::kSmem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  fill_pdl_attr(cfg, attr);
  const cudaError_t e = cudaLaunchKernelEx(&cfg, mha_prefill_tc_kernel<D>, mq, mk, mv, p);
  if (e != cudaSuccess && getenv("IRON_DEBUG")) fprintf(stderr, "mha_prefill_tc<%d>: %s\n", D, cudaGetErrorString(e));
  return e == cudaSuccess ? IRON_OK : IRON_ERR_LAUNCH;
}

// The tensor-memory form of the prompt-chunk attention; bounds known on the host.  Returns
// IRON_ERR_UNSUPPORTED for layouts a tensor map cannot describe (the caller then takes the
// warp-MMA kernel).
int mha_prefill_tc(const void* Q, const void* K, const void* V, void* O, int batch, int H, int G, int D,
                   int q_rows, long long q_batch_stride, long long q_row_stride, long long q_head_stride,
                   long long o_batch_stride, long long o_row_stride, long long o_head_stride,
                   long long kv_batch_stride, long long kv_row_stride, long long kv_head_stride, int q_tokens,
                   int kv_tokens, int causal, int window, float scale, int* d_status, cudaStream_t stream) {
  if (q_tokens <= 0 || kv_tokens <= 0 || !(scale > 0.f)) return IRON_ERR_UNSUPPORTED;
  if ((causal || window >= 0) && kv_tokens < q_tokens) return IRON_ERR_UNSUPPORTED;
  CUtensorMap mq, mk, mv;
  if (!tc_map(&mq, Q, D, H, q_tokens, batch, q_head_stride, q_row_stride, q_batch_stride) ||
      !tc_map(&mk, K, D, G, kv_tokens, batch, kv_head_stride, kv_row_stride, kv_batch_stride) ||
      !tc_map(&mv, V, D, G, kv_tokens, batch, kv_head_stride, kv_row_stride, kv_batch_stride))
    return IRON_ERR_UNSUPPORTED;
  PrefillTcParams p = {};
  p.O = (__nv_bfloat16*)O;
  p.o_batch_stride = o_batch_stride; p.o_row_stride = o_row_stride; p.o_head_stride = o_head_stride;
  p.H = H; p.G = G; p.batch = batch; p.q_rows = q_rows; p.q_tokens = q_tokens; p.kv_tokens = kv_tokens;
  p.causal = causal; p.window = window;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.status = d_status;
#ifdef TC_TRACE
  { static long long* tb = nullptr; if (!tb) { cudaMalloc(&tb, 8 * 64 * 8); cudaMemset(tb, 0, 8 * 64 * 8); } p.trace = tb; g_tc_trace = tb; }
#endif
  if (D == 64) return launch_prefill_tc<64>(mq, mk, mv, p, batch, stream);
  return launch_prefill_tc<128>(mq, mk, mv, p, batch, stream);
}

}  // namespace iron

#ifdef TC_TRACE
extern "C" void iron_tc_trace(long long* host_out) { cudaMemcpy(host_out, iron::g_tc_trace, 8 * 64 * 8, cudaMemcpyDeviceToHost); }
#endif
