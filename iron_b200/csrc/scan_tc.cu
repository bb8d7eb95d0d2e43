// Mamba2's selective scan in its chunked ("state-space dual") form on tcgen05 / tensor memory.
//
// With a_t = step_t * A (<= 0) and cum_t the running sum of a over a chunk of Q = 128 rows,
//
//   y_t     = sum_{j <= t} exp(cum_t - cum_j) step_j (C_t . B_j) x_j  +  exp(cum_t) C_t . S_prev  +  D x_t
//   S_next  = exp(cum_Q) S_prev  +  sum_j exp(cum_Q - cum_j) step_j  x_j (x) B_j
//
// so a chunk is four matrix products (iron/operators/selective_scan.py:46 is the recurrence):
//   P1  scores   S  (Q x Q)  = C B^T                     over the N = 128 states
//   P2  intra    Y  (Q x P)  = M X,  M = masked, decayed scores
//   P3  read-out Z  (Q x P)  = C S_prev^T                over the states
//   P4  update   dS^T (N x P) = B^T X_w,  X_w = x_j w_j   over the chunk's rows
// One CTA owns one (sequence, head), P = 64.  Every product is a 128-row tcgen05.mma with its
// accumulator in tensor memory; x, B and C arrive by TMA (128-byte swizzle) and are operands as
// they lie: C and B K-major for P1, B again as the M-major A operand of P4, x as the N-major B
// operand of P2.  The float32 operands -- M, X_w and the carried state -- enter as a bf16 head AND
// a bf16 remainder (two accumulating products), so every product keeps float32's accuracy: X_w
// and the state written to shared memory in the operand layout, M stored to tensor memory, from
// where P2 takes it as its A operand.  A compute thread owns one row: row t
// of the scores, of y and of x; row n of the transposed state, whose 64 float32 values stay in
// its registers from chunk to chunk.
//
// Roles (512 threads).  Warps 0-3, the state warps: a chunk's steps and their running sum,
// published one chunk ahead, then S = decay S + dS and its split -> [P3 of the next chunk].
// Warps 4-11, the row warps, two per tensor-memory lane quarter: the masked scores of columns
// 0-63 / 64-127, written over the scores in tensor memory -> [P2], then 32 of the row's 64
// outputs each; the four of them with the least below the diagonal also make the next chunk's
// weighted rows -> [P4].  Warps 12, 13 and 15 issue the MMAs (a product family each: these
// products are small, and what they wait for is their issue), warp 14 the TMA loads.  One warp
// alone on a scheduler runs these dependent chains at a fifth of an instruction per clock; three
// or four a scheduler overlap them.
// B and C are single-buffered and reloaded as soon as their last product has read them (a
// commit), early in the chunk; x is double-buffered.  Every wait is bounded (2 s ->
// IRON_ERR_TIMEOUT in the status word); the state warps leave their loop together.
#include <cuda.h>

#include "scan.cuh"
#include "tc.cuh"

namespace iron {

constexpr int kTcQ = 128;            // rows per chunk
constexpr int kTcP = 64;             // head_dim
constexpr int kTcNs = 128;           // states
constexpr int kTcSub = 16384;        // one 128-row x 128-byte swizzled tile
constexpr int kTcThreads = 512;      // 12 compute warps, three MMA warps, the TMA warp
constexpr int kTcMmaWarp = 15, kTcMmaWarp2 = 13, kTcTmaWarp = 14, kTcMmaWarp3 = 12;   // P2 | P3, P4 | TMA | P1

struct SsdTcSmem {
  static constexpr int kX = 0;                         // 2 x (Q x P)            x of chunk c, c + 1
  static constexpr int kB = kX + 2 * kTcSub;           // 2 tiles: states 0-63, 64-127
  static constexpr int kC = kB + 2 * kTcSub;
  static constexpr int kXwHi = kC + 2 * kTcSub;        // the weighted rows (Q x P), head and remainder
  static constexpr int kXwLo = kXwHi + kTcSub;
  static constexpr int kShi = kXwLo + kTcSub;          // the state, transposed (N x P), head and remainder
  static constexpr int kSlo = kShi + kTcSub;
  static constexpr int kF = kSlo + kTcSub;             // cum and g of three chunks (2 x 3 x Q floats); 2 x 4 warp totals
  static constexpr int kBars = kF + (6 * kTcQ + 8) * 4;
  static constexpr int kNumBars = 20;
  static constexpr int kTotal = kBars + kNumBars * 8 + 16 + 1024;   // + tmem slot, abort flag, alignment slack
};

__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* map, int x, int y, int z, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(x), "r"(y), "r"(z), "r"(smem_u32(bar))
      : "memory");
}
// bf16 x bf16 -> f32, M = 128; operands K-major unless their flag says M-/N-major.
__host__ __device__ constexpr uint32_t ssd_idesc(int n, bool a_m_major, bool b_n_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((a_m_major ? 1u : 0u) << 15) | ((b_n_major ? 1u : 0u) << 16) |
         ((uint32_t)(n >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
}
// All 128 compute threads meet; each learns whether every one of them is still fine.
__device__ __forceinline__ bool compute_sync_all_ok(bool ok) {
  uint32_t r;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.b32 p, %1, 0;\n\t"
      "barrier.red.and.pred q, 1, 128, p;\n\t"
      "selp.u32 %0, 1, 0, q;\n\t}"
      : "=r"(r) : "r"((uint32_t)ok) : "memory");
  return r != 0;
}
// A float32 pair as a bf16 head and the bf16 of what the head left over, in six instructions on the
// integer and float pipes: the head is the value cut to its upper 16 bits (the remainder is then
// exact in float32), the remainder is cut the same way, so head + remainder is within 2^-14 of
// the value (plain bf16: 2^-8).  The conversion instruction would round both to nearest, but it
// shares the special-function unit with the exponentials, and these kernels' compute warps are
// bound by the instructions they issue: 100 to 130 pairs a row and chunk.
__device__ __forceinline__ void ssd_split(float v0, float v1, uint32_t& hi, uint32_t& lo) {
  const uint32_t u0 = __float_as_uint(v0), u1 = __float_as_uint(v1);
  hi = __byte_perm(u0, u1, 0x7632);
  const float l0 = v0 - __uint_as_float(u0 & 0xffff0000u), l1 = v1 - __uint_as_float(u1 & 0xffff0000u);
  lo = __byte_perm(__float_as_uint(l0), __float_as_uint(l1), 0x7632);
}
__device__ __forceinline__ float ssd_ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float ssd_lg2(float x) {
  float y;
  asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// softplus(v) = max(v, 0) + log1p(exp(-|v|)) in a dozen instructions: e = exp(-|v|) <= 1 on the
// hardware's exp2, and log1p(e) = 2 atanh(z), z = e / (2 + e) <= 1/3, as its odd series up to z^13
// (the next term is below 2e-8 of the value).
__device__ __forceinline__ float ssd_softplus(float v) {
  const float e = ssd_ex2(-fabsf(v) * 1.4426950408889634f);
  const float z = __fdividef(e, 2.0f + e), w = z * z;
  float poly = fmaf(w, 1.0f / 13.0f, 1.0f / 11.0f);
  poly = fmaf(w, poly, 1.0f / 9.0f);
  poly = fmaf(w, poly, 1.0f / 7.0f);
  poly = fmaf(w, poly, 1.0f / 5.0f);
  poly = fmaf(w, poly, 1.0f / 3.0f);
  poly = fmaf(w, poly, 1.0f);
  return fmaxf(v, 0.f) + 2.0f * z * poly;
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
// 16 registers of this thread into 16 consecutive columns of its tensor-memory lane.
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// The same MMA with its A operand in tensor memory: row = lane, two bf16 of K per 32-bit column.
__device__ __forceinline__ void tcgen05_mma_bf16_ta(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                                    uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// The MMAs as the issuing thread sees them: a descriptor is two 32-bit halves, and a K step moves
// only the low one (the 14-bit address field, in 16-byte units, never carries), so a step costs
// the issuer one add.  It issues ~one instruction per ten clocks next to three compute warps on
// its scheduler, and these products are small: what they wait for is their issue.
__device__ __forceinline__ void ssd_mma_ss(uint32_t d, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo, uint32_t b_hi,
                                           uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
      "setp.ne.b32 p, %6, 0;\n\t"
      "mov.b64 da, {%1, %2};\n\t"
      "mov.b64 db, {%3, %4};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, p;\n\t}"
      ::"r"(d), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void ssd_mma_ts(uint32_t d, uint32_t a_tmem, uint32_t b_lo, uint32_t b_hi, uint32_t idesc,
                                           uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 db;\n\t"
      "setp.ne.b32 p, %5, 0;\n\t"
      "mov.b64 db, {%2, %3};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %4, p;\n\t}"
      ::"r"(d), "r"(a_tmem), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Row r's 16-byte chunk c of a 128-byte-swizzled tile.
__device__ __forceinline__ uint4* tile_chunk(uint8_t* tile, int r, int c) {
  return reinterpret_cast<uint4*>(tile + r * 128 + ((c ^ (r & 7)) << 4));
}

#ifdef SSD_TC_TRACE
__device__ long long g_ssd_trace[4 * 64 * 16];
#define SSD_MMARK(i) if (h == 0 && b == 0 && c < 64) g_ssd_trace[(3 * 64 + c) * 16 + (i)] = clock64();
#define SSD_MARK(who, i) if (r == 127 && h == 0 && b == 0 && c < 64) g_ssd_trace[((who) * 64 + c) * 16 + (i)] = clock64();
#else
#define SSD_MARK(who, i)
#define SSD_MMARK(i)
#endif

// One copy of the bounded wait for the whole kernel: fifteen warps run five different roles out of
// one instruction cache, and the code's size is what they wait for first.
__device__ __noinline__ bool ssd_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  return mbar_wait_relaxed(bar, parity, abort_flag, 20);
}

enum {
  BAR_XFULL = 0,   // [2]  TMA: x of a chunk
  BAR_BFULL = 2, BAR_CFULL = 3,
  BAR_XFREE = 4,   // [2]  compute (128): the chunk's output rows are done with x
  BAR_BFREE = 6, BAR_CFREE = 7,          // commits: the last product that reads the tile is done
  BAR_S = 8, BAR_Z = 9, BAR_D = 10, BAR_Y = 11,   // commits: an accumulator is whole
  BAR_XW = 12, BAR_M = 13, BAR_STATE = 14, BAR_E = 15,  // compute: an operand is written / the outputs are read
  BAR_SCAN = 16    // [3]  compute: a chunk's running sums are published (chunk c uses barrier and buffer c % 3)
};

__global__ void __launch_bounds__(kTcThreads, 1)
ssd_scan_tc_kernel(const __grid_constant__ CUtensorMap map_xbc, const ScanParams p, int* status) {
  using L = SsdTcSmem;
  constexpr int Q = kTcQ, P = kTcP, N = kTcNs;
  extern __shared__ uint8_t ssd_tc_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(ssd_tc_raw) + 1023) & ~uintptr_t(1023));
  float* s_cum = reinterpret_cast<float*>(smem + L::kF);
  float* s_g = s_cum + 3 * Q;
  float* s_tot = s_g + 3 * Q;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBars);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + L::kNumBars);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int h = blockIdx.x, b = blockIdx.y;
  const int grp = h / (p.H / p.G);
  const int inner = p.H * P;
  const int chunks = (p.rows + Q - 1) / Q;

  if (tid == 0) {
    for (int i = 0; i < L::kNumBars; ++i) {
      int count = 1;                                                        // a TMA transaction or a commit
      if (i == BAR_STATE || (i >= BAR_SCAN && i < BAR_SCAN + 3)) count = 128;   // the state warps
      if (i == BAR_BFREE || i == BAR_CFREE) count = 2;                        // a commit from each MMA warp that reads the tile
      if (i == BAR_XW) count = 128;                                           // the four row warps that weight x
      if (i == BAR_XFREE || i == BAR_XFREE + 1 || i == BAR_M || i == BAR_E) count = 256;   // the row warps
      mbar_init(bars + i, count);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_xbc) : "memory");
  }
  if (warp == kTcMmaWarp) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // Tensor memory, 512 columns: the scores, which each row overwrites in place with its masked scores
  // as bf16 pairs (per 32 columns: 16 of heads, 16 of remainders); Z and dS with the heads' and the
  // remainders' products side by side (one 128-column product each: the state's two tiles, and the
  // weighted rows' two, are each one N-major operand), added when read; Y and the remainders' Y.
  constexpr uint32_t kColS = 0, kColZ = 128, kColD = 256, kColY = 384, kColY2 = 448;

  pdl_launch();
  pdl_wait();
  int valid = p.d_valid ? min(*p.d_valid, p.rows) : p.valid;
  valid = max(valid, 0);

  if (warp == kTcTmaWarp) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      const int col_x = h * P, col_b = inner + grp * N, col_c = inner + (p.G + grp) * N;
      for (int c = 0; c < chunks; ++c) {
        const int row = c * Q, s = c & 1;
        // x: the buffer's last reader was the output step of chunk c - 2
        if (c >= 2 && !ssd_wait(bars + BAR_XFREE + s, ((c - 2) >> 1) & 1, abort_flag)) break;
        mbar_expect_tx(bars + BAR_XFULL + s, kTcSub);
        tma_load_3d(smem + L::kX + s * kTcSub, &map_xbc, col_x, row, b, bars + BAR_XFULL + s);
        if (c >= 1 && !ssd_wait(bars + BAR_CFREE, (c - 1) & 1, abort_flag)) break;
        mbar_expect_tx(bars + BAR_CFULL, 2 * kTcSub);
        tma_load_3d(smem + L::kC, &map_xbc, col_c, row, b, bars + BAR_CFULL);
        tma_load_3d(smem + L::kC + kTcSub, &map_xbc, col_c + 64, row, b, bars + BAR_CFULL);
        if (c >= 1 && !ssd_wait(bars + BAR_BFREE, (c - 1) & 1, abort_flag)) break;
        mbar_expect_tx(bars + BAR_BFULL, 2 * kTcSub);
        tma_load_3d(smem + L::kB, &map_xbc, col_b, row, b, bars + BAR_BFULL);
        tma_load_3d(smem + L::kB + kTcSub, &map_xbc, col_b + 64, row, b, bars + BAR_BFULL);
      }
    }
  } else if (warp == kTcMmaWarp || warp == kTcMmaWarp2 || warp == kTcMmaWarp3) {
    // ---------------- MMA issuers ----------------
    // Three of them, one product family each -- P2 | P3 and P4 | P1 -- because these products are
    // small and what they wait for is their issue: alone, a thread issues one 64-column product per
    // 46 clocks (32 of arithmetic), next to busy compute warps on its scheduler one per ~140.  P2
    // is the one the rows wait for, so its issuer sits on the scheduler of the lane quarter whose
    // row warps have the most to mask and nothing to do once they have signalled (warp 15, with
    // warps 3, 7 and 11).  And the products are as wide as they can be:
    // head and remainder of the state (and of the weighted rows) are the two 64-column halves of
    // ONE N-major operand, 128 columns a product.
    if (lane == 0) {
      constexpr uint32_t idesc_s = ssd_idesc(128, false, false);   // C (K-major) x B (K-major)
      constexpr uint32_t idesc_y = ssd_idesc(P, false, true);      // M (tensor memory) x X (N-major)
      constexpr uint32_t idesc_z = ssd_idesc(128, false, true);    // C (K-major) x state, head | remainder (N-major)
      constexpr uint32_t idesc_d = ssd_idesc(128, true, true);     // B (M-major) x X_w, head | remainder (N-major)
      auto lo32 = [](uint64_t d) { return (uint32_t)d; };
      auto hi32 = [](uint64_t d) { return (uint32_t)(d >> 32); };
      const uint64_t c_desc = make_desc(smem_u32(smem + L::kC), 16, 1024);
      const uint64_t b_desc = make_desc(smem_u32(smem + L::kB), 16, 1024);
      const uint64_t bt_desc = make_desc(smem_u32(smem + L::kB), kTcSub, 1024);   // 64-state chunks one tile apart
      const uint64_t st_desc = make_desc(smem_u32(smem + L::kShi), kTcSub, 1024);   // head tile, remainder tile
      const uint64_t xw_desc = make_desc(smem_u32(smem + L::kXwHi), kTcSub, 1024);
      const uint64_t x_desc0 = make_desc(smem_u32(smem + L::kX), kTcSub, 1024);
      // K-major operand, step k of 8: tile k / 4, 32 bytes per step; M-/N-major: 16 rows of 128 bytes per step
      auto kmaj = [](int k) { return (uint32_t)(((k >> 2) * kTcSub + (k & 3) * 32) >> 4); };
      auto nmaj = [](int k) { return (uint32_t)((k * 16 * 128) >> 4); };
      if (warp == kTcMmaWarp) {
#pragma unroll 1
        for (int c = 0; c < chunks; ++c) {
          const uint32_t ph = c & 1;
          const uint32_t x_lo = lo32(x_desc0) + (uint32_t)(((c & 1) * kTcSub) >> 4);
          // P2: the masked scores (heads, remainders: two accumulators, step by step in turn) times x;
          // Y is free once the last chunk's output rows have been read
          if (!ssd_wait(bars + BAR_M, ph, abort_flag)) break;
          if (c >= 1 && !ssd_wait(bars + BAR_E, (c - 1) & 1, abort_flag)) break;
          if (!ssd_wait(bars + BAR_XFULL + (c & 1), (c >> 1) & 1, abort_flag)) break;
          tcgen05_fence_after();
          SSD_MMARK(2)
#pragma unroll
          for (int k = 0; k < Q / 16; ++k) {
            const uint32_t m_col = tmem_base + kColS + 32 * (k >> 1) + 8 * (k & 1);
            ssd_mma_ts(tmem_base + kColY, m_col, x_lo + nmaj(k), hi32(x_desc0), idesc_y, k != 0);
            ssd_mma_ts(tmem_base + kColY2, m_col + 16, x_lo + nmaj(k), hi32(x_desc0), idesc_y, k != 0);
          }
          SSD_MMARK(3)
          tcgen05_commit(bars + BAR_Y);
        }
      } else if (warp == kTcMmaWarp2) {
#pragma unroll 1
        for (int c = 0; c < chunks; ++c) {
          const uint32_t ph = c & 1;
          // P3, the read-out of the carried state (written at the end of the last chunk), and P4, the
          // state's update, transposed, step by step in turn.  Z is free once the last chunk's output
          // rows have been read, dS once the state warps have written the state.
          if (!ssd_wait(bars + BAR_BFULL, ph, abort_flag) || !ssd_wait(bars + BAR_CFULL, ph, abort_flag)) break;
          if (!ssd_wait(bars + BAR_STATE, ph, abort_flag)) break;
          if (c >= 1 && !ssd_wait(bars + BAR_E, (c - 1) & 1, abort_flag)) break;
          if (!ssd_wait(bars + BAR_XW, ph, abort_flag)) break;
          tcgen05_fence_after();
          SSD_MMARK(0)
#pragma unroll
          for (int k = 0; k < N / 16; ++k) {
            ssd_mma_ss(tmem_base + kColZ, lo32(c_desc) + kmaj(k), hi32(c_desc), lo32(st_desc) + nmaj(k), hi32(st_desc),
                       idesc_z, k != 0);
            ssd_mma_ss(tmem_base + kColD, lo32(bt_desc) + nmaj(k), hi32(bt_desc), lo32(xw_desc) + nmaj(k), hi32(xw_desc),
                       idesc_d, k != 0);
          }
          SSD_MMARK(1)
          tcgen05_commit(bars + BAR_Z);
          tcgen05_commit(bars + BAR_D);
          tcgen05_commit(bars + BAR_CFREE);
          tcgen05_commit(bars + BAR_BFREE);
        }
      } else {
#pragma unroll 1
        for (int c = 0; c < chunks; ++c) {
          const uint32_t ph = c & 1;
          // P1: the scores.  Their columns held the last chunk's masked scores, which P2 of that chunk
          // must have read.
          if (!ssd_wait(bars + BAR_BFULL, ph, abort_flag) || !ssd_wait(bars + BAR_CFULL, ph, abort_flag)) break;
          if (c >= 1 && !ssd_wait(bars + BAR_Y, (c - 1) & 1, abort_flag)) break;
          tcgen05_fence_after();
#pragma unroll
          for (int k = 0; k < N / 16; ++k)
            ssd_mma_ss(tmem_base + kColS, lo32(c_desc) + kmaj(k), hi32(c_desc), lo32(b_desc) + kmaj(k), hi32(b_desc),
                       idesc_s, k != 0);
          tcgen05_commit(bars + BAR_S);
          tcgen05_commit(bars + BAR_CFREE);
          tcgen05_commit(bars + BAR_BFREE);
        }
      }
    }
  } else if (warp < 4) {
    // ---------------- the state warps: thread r owns row r of x and row r of the transposed state ----------------
    const int r = tid;
    const uint32_t lane_base = tmem_base + ((uint32_t)(warp * 32) << 16);
    const float dt_bias = p.head[h * 3], A = p.head[h * 3 + 1];
    const __nv_bfloat16* dtp = p.dt + (size_t)b * p.dt_batch + h;
    auto proxy_fence = [] { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); };

    float st[P];      // S[q][r] for every q
    {
      const float* src = p.state ? p.state + (size_t)b * p.state_batch + (size_t)h * P * N : nullptr;
#pragma unroll
      for (int q = 0; q < P; ++q) st[q] = src ? src[(size_t)q * N + r] : 0.f;
    }
    // Shared-memory loads cannot move across shared-memory stores (the compiler cannot tell the tiles
    // apart), so a step reads what it needs, computes in registers, then stores; in halves, for the
    // registers' sake.
    auto write_state = [&]() {
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        uint4 hi[4], lo[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float* v = st + 32 * half + 8 * q;
          ssd_split(v[0], v[1], hi[q].x, lo[q].x);
          ssd_split(v[2], v[3], hi[q].y, lo[q].y);
          ssd_split(v[4], v[5], hi[q].z, lo[q].z);
          ssd_split(v[6], v[7], hi[q].w, lo[q].w);
        }
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          *tile_chunk(smem + L::kShi, r, 4 * half + q) = hi[q];
          *tile_chunk(smem + L::kSlo, r, 4 * half + q) = lo[q];
        }
      }
      proxy_fence();
      mbar_arrive(bars + BAR_STATE);
    };
    // The running sum of chunk c is made while chunk c - 1's update product is in flight (it needs
    // only dt), and published in buffer c % 3: the row warps may still be reading chunk c - 2's.
    bool ok = true;
    float dt_next = r < p.rows ? __bfloat162float(dtp[(size_t)r * p.H]) : 0.f;
    auto publish_scan = [&](int c) -> float {      // returns the chunk's decay exp(cum_Q); leaves `ok` the same in every thread
      const int t = c * Q + r;
      const float step = t < valid ? ssd_softplus(dt_next + dt_bias) : 0.f;   // rows past the bound: a = 0, step = 0
      if (c + 1 < chunks && t + Q < p.rows) dt_next = __bfloat162float(dtp[(size_t)(t + Q) * p.H]);
      float cum = step * A;
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        const float u = __shfl_up_sync(0xffffffffu, cum, off);
        if (lane >= off) cum += u;
      }
      float* tot = s_tot + 4 * (c & 1);
      if (lane == 31) tot[warp] = cum;
      ok = compute_sync_all_ok(ok);
      float total = 0.f;
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        const float tw = tot[w];
        if (w < warp) cum += tw;
        total += tw;
      }
      // from here the sums are in units of log 2 (every decay is one ex2); g = the sum less log2(step),
      // so that a masked score is S ex2(cum_t - g_j) and a row's weight ex2(cum_Q - g_j); a row past
      // the bound has step 0, g = +inf and weight 0
      constexpr float kLog2e = 1.4426950408889634f;
      cum *= kLog2e;
      total *= kLog2e;
      const int buf = (c % 3) * Q;
      s_cum[buf + r] = cum;
      s_g[buf + r] = cum - ssd_lg2(step);
      mbar_arrive(bars + BAR_SCAN + c % 3);
      return ssd_ex2(total);
    };
    // Iteration -1 publishes the first chunk's sums and writes the incoming state; iteration c
    // publishes chunk c + 1's (one call site each: the kernel's code must stay small).
    float decay = 0.f;
    bool all_ok = true;                                // the same in every state thread: they leave together
#pragma unroll 1
    for (int c = -1; c < chunks && all_ok; ++c) {
      const uint32_t ph = c & 1;
      float decay_next = 0.f;
      SSD_MARK(0, 0)
      if (c + 1 < chunks) {
        decay_next = publish_scan(c + 1);
        all_ok = ok;
        if (!all_ok) break;
      }
      if (c >= 0) {
        // ---- S = exp(cum_Q) S + dS, split for the next chunk's read-out (P3 has read the old one) ----
        SSD_MARK(0, 1)
        ok = ok && ssd_wait(bars + BAR_D, ph, abort_flag);
        tcgen05_fence_after();
        SSD_MARK(0, 4)
#pragma unroll
        for (int part = 0; part < 4; ++part) {
          uint32_t v[16], v2[16];
          tmem_ld16(lane_base + kColD + 16 * part, v);
          tmem_ld16(lane_base + kColD + 64 + 16 * part, v2);     // the remainders' product
          tmem_ld_wait();
#pragma unroll
          for (int q = 0; q < 16; ++q)
            st[16 * part + q] = fmaf(decay, st[16 * part + q], __uint_as_float(v[q]) + __uint_as_float(v2[q]));
        }
        tcgen05_fence_before();
        SSD_MARK(0, 5)
        ok = ok && ssd_wait(bars + BAR_Z, ph, abort_flag);
        SSD_MARK(0, 6)
      }
      write_state();
      SSD_MARK(0, 7)
      decay = decay_next;
    }
    if (p.final_state && ok) {
      float* dst = p.final_state + (size_t)b * p.state_batch + (size_t)h * P * N;
#pragma unroll
      for (int q = 0; q < P; ++q) dst[(size_t)q * N + r] = st[q];
    }
  } else {
    // ---------------- the row warps: thread r owns row r of the scores and of y; warps 4-7 take score
    // columns 0-63 and output columns 0-31, warps 8-11 columns 64-127 and 32-63 ----------------
    const int r = tid & 127, quarter = warp & 3, side = (warp - 4) >> 2;
    const uint32_t lane_base = tmem_base + ((uint32_t)(quarter * 32) << 16);
    const float Dh = p.head[h * 3 + 2];
    __nv_bfloat16* yb = p.y + (size_t)b * p.y_batch + (size_t)h * P + 32 * side;

    // 32 columns of this row's scores -> masked, decayed, split -> the A operand of P2 in tensor memory
    // (this row's lane; a 32-bit column holds the bf16 of columns j, j + 1)
    auto mask_batch = [&](int bq, float cum_r, const float* g_all) {
      uint32_t hi[16], lo[16];
      if (bq > quarter) {      // wholly above the diagonal for every row of this warp
#pragma unroll
        for (int q = 0; q < 16; ++q) hi[q] = lo[q] = 0u;
      } else {
        uint32_t v[32];
        tmem_ld32(lane_base + kColS + 32 * bq, v);
        float4 gj[8];
#pragma unroll
        for (int q = 0; q < 8; ++q) gj[q] = *reinterpret_cast<const float4*>(g_all + 32 * bq + 4 * q);
        tmem_ld_wait();
        const bool diagonal = bq == quarter;      // only the warp's own batch crosses the diagonal
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          const int j = 32 * bq + 4 * q;
          const float g4[4] = {gj[q].x, gj[q].y, gj[q].z, gj[q].w};
          float m[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            m[e] = __uint_as_float(v[4 * q + e]) * ssd_ex2(cum_r - g4[e]);
            if (diagonal && j + e > r) m[e] = 0.f;
          }
          ssd_split(m[0], m[1], hi[2 * q], lo[2 * q]);
          ssd_split(m[2], m[3], hi[2 * q + 1], lo[2 * q + 1]);
        }
      }
      // in place: the 32 score columns become 16 columns of heads and 16 of remainders
      tmem_st16(lane_base + kColS + 32 * bq, hi);
      tmem_st16(lane_base + kColS + 32 * bq + 16, lo);
    };

    // The four row warps with the least below the diagonal (warps 8 and 9: nothing; 4 and 10: one
    // batch) make the weighted rows x_j w_j, w_j = exp(cum_Q - cum_j) step_j: a row a thread, one
    // chunk ahead (x, the running sums and the buffer -- once P4 has read the last ones -- are all
    // there early), so that P4 of a chunk can start with the chunk.
    const int xw_rows = warp == 8 ? 0 : warp == 9 ? 32 : warp == 4 ? 64 : warp == 10 ? 96 : -1;
    const bool weights_x = xw_rows >= 0;
    auto proxy_fence = [] { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); };
    bool ok = true;
    auto weigh_rows = [&](int c) {
      const int s = c & 1;
      uint8_t* x_tile = smem + L::kX + s * kTcSub;
      ok = ok && ssd_wait(bars + BAR_SCAN + c % 3, (c / 3) & 1, abort_flag);
      ok = ok && ssd_wait(bars + BAR_XFULL + s, (c >> 1) & 1, abort_flag);
      if (c >= 1) ok = ok && ssd_wait(bars + BAR_D, (c - 1) & 1, abort_flag);
      const float* g_all = s_g + (c % 3) * Q;
      const float total = s_cum[(c % 3) * Q + Q - 1];
      {
        const int j = xw_rows + lane;
        const float w_j = ssd_ex2(total - g_all[j]);
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          uint4 xv[4], hi[4], lo[4];
#pragma unroll
          for (int q = 0; q < 4; ++q) xv[q] = *tile_chunk(x_tile, j, 4 * half + q);
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            ssd_split(bf16_lo(xv[q].x) * w_j, bf16_hi(xv[q].x) * w_j, hi[q].x, lo[q].x);
            ssd_split(bf16_lo(xv[q].y) * w_j, bf16_hi(xv[q].y) * w_j, hi[q].y, lo[q].y);
            ssd_split(bf16_lo(xv[q].z) * w_j, bf16_hi(xv[q].z) * w_j, hi[q].z, lo[q].z);
            ssd_split(bf16_lo(xv[q].w) * w_j, bf16_hi(xv[q].w) * w_j, hi[q].w, lo[q].w);
          }
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            *tile_chunk(smem + L::kXwHi, j, 4 * half + q) = hi[q];
            *tile_chunk(smem + L::kXwLo, j, 4 * half + q) = lo[q];
          }
        }
      }
      proxy_fence();
      mbar_arrive(bars + BAR_XW);
    };
#pragma unroll 1
    for (int c = -1; c < chunks && ok; ++c) {
      // iteration -1 only weighs the first chunk's rows (one call site: the code must stay small)
      const uint32_t ph = c & 1;
      const int s = c & 1, t = c * Q + r;
      uint8_t* x_tile = smem + L::kX + s * kTcSub;
      float cum_r = 0.f;
      if (c >= 0) {
        SSD_MARK(1 + side, 0)
        ok = ok && ssd_wait(bars + BAR_SCAN + c % 3, (c / 3) & 1, abort_flag);
        const float* g_all = s_g + (c % 3) * Q;
        cum_r = s_cum[(c % 3) * Q + r];
        // ---- the masked scores of this side's columns -> P2 ----
        SSD_MARK(1 + side, 1)
        ok = ok && ssd_wait(bars + BAR_S, ph, abort_flag);
        tcgen05_fence_after();
        SSD_MARK(1 + side, 2)
#pragma unroll 1
        for (int i = 0; i < 2; ++i) mask_batch(2 * side + i, cum_r, g_all);
        tmem_st_wait();
        tcgen05_fence_before();
        mbar_arrive(bars + BAR_M);
        SSD_MARK(1 + side, 3)
      }
      if (weights_x && c + 1 < chunks) weigh_rows(c + 1);   // after the signal: P2 does not wait for this
      if (c < 0) continue;

      // ---- y_r = Y_r + exp(cum_r) Z_r + D x_r, this side's 32 columns ----
      ok = ok && ssd_wait(bars + BAR_XFULL + s, (c >> 1) & 1, abort_flag);
      const float e_r = ssd_ex2(cum_r);
      SSD_MARK(1 + side, 4)
      ok = ok && ssd_wait(bars + BAR_Z, ph, abort_flag);
      SSD_MARK(1 + side, 5)
      ok = ok && ssd_wait(bars + BAR_Y, ph, abort_flag);
      tcgen05_fence_after();
      SSD_MARK(1 + side, 6)
#pragma unroll 1
      for (int hh = 0; hh < 2; ++hh) {          // 16 of this side's 32 columns at a time
        const int col = 32 * side + 16 * hh;
        uint4 xr[2];
#pragma unroll
        for (int q = 0; q < 2; ++q) xr[q] = *tile_chunk(x_tile, r, 4 * side + 2 * hh + q);
        uint32_t y1[16], y2[16], z1[16], z2[16];
        tmem_ld16(lane_base + kColY + col, y1);
        tmem_ld16(lane_base + kColY2 + col, y2);
        tmem_ld16(lane_base + kColZ + col, z1);
        tmem_ld16(lane_base + kColZ + 64 + col, z2);       // the remainders' product
        tmem_ld_wait();
        if (hh == 0) { SSD_MARK(1 + side, 8) }
        uint4 out[2];
#pragma unroll
        for (int q = 0; q < 2; ++q) {
          const uint4 xq = xr[q];
          const uint32_t xw[4] = {xq.x, xq.y, xq.z, xq.w};
          uint32_t o[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int i = 8 * q + 2 * e;
            const float ya = __uint_as_float(y1[i]) + __uint_as_float(y2[i]);
            const float yc = __uint_as_float(y1[i + 1]) + __uint_as_float(y2[i + 1]);
            const float za = __uint_as_float(z1[i]) + __uint_as_float(z2[i]);
            const float zc = __uint_as_float(z1[i + 1]) + __uint_as_float(z2[i + 1]);
            const float v0 = fmaf(Dh, bf16_lo(xw[e]), fmaf(e_r, za, ya));
            const float v1 = fmaf(Dh, bf16_hi(xw[e]), fmaf(e_r, zc, yc));
            o[e] = t < valid ? pack_bf16x2(v0, v1) : 0u;
          }
          out[q] = make_uint4(o[0], o[1], o[2], o[3]);
        }
        if (t < p.rows) {
#pragma unroll
          for (int q = 0; q < 2; ++q) *reinterpret_cast<uint4*>(yb + (size_t)t * inner + 16 * hh + 8 * q) = out[q];
        }
      }
      SSD_MARK(1 + side, 9)
      tcgen05_fence_before();
      mbar_arrive(bars + BAR_E);
      mbar_arrive(bars + BAR_XFREE + s);
      SSD_MARK(1 + side, 7)
    }
  }

  tcgen05_fence_before();
  __syncthreads();
  if (tid == 0 && *abort_flag && status) *status = IRON_ERR_TIMEOUT;
  if (warp == kTcMmaWarp) {
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
  }
}

// ---- host side ---------------------------------------------------------------
typedef CUresult (*SsdEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static SsdEncodeFn ssd_encode() {
  static SsdEncodeFn fn = nullptr;
  if (!fn) {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<SsdEncodeFn>(sym);
  }
  return fn;
}

int launch_ssd_tc(const ScanParams& p, int batch, cudaStream_t stream, int* d_status) {
  SsdEncodeFn fn = ssd_encode();
  if (!fn || p.P != kTcP || (p.width & 7)) return IRON_ERR_UNSUPPORTED;
  // (column, row, sequence) over the call's x | B | C rows; boxes of 64 columns x 128 rows, rows past the
  // call read as zeros
  CUtensorMap map;
  const cuuint64_t dims[3] = {(cuuint64_t)p.width, (cuuint64_t)p.rows, (cuuint64_t)batch};
  const cuuint64_t strides[2] = {(cuuint64_t)p.width * 2, (cuuint64_t)(batch > 1 ? p.xbc_batch : (long long)p.width * p.rows) * 2};
  const cuuint32_t box[3] = {64, (cuuint32_t)kTcQ, 1};
  const cuuint32_t elem[3] = {1, 1, 1};
  if (fn(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<__nv_bfloat16*>(p.xbc), dims, strides, box, elem,
         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return IRON_ERR_UNSUPPORTED;
  static DeviceOnce configured;   // the attribute is per device
  if (!configured.done()) {
    if (cudaFuncSetAttribute(ssd_scan_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SsdTcSmem::kTotal) !=
        cudaSuccess)
      return IRON_ERR_LAUNCH;
    configured.mark();
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(p.H, batch);
  cfg.blockDim = dim3(kTcThreads);
  cfg.dynamicSmemBytes = SsdTcSmem::kTotal;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  fill_pdl_attr(cfg, attr);
  return cudaLaunchKernelEx(&cfg, ssd_scan_tc_kernel, map, p, d_status) == cudaSuccess ? IRON_OK : IRON_ERR_LAUNCH;
}

}  // namespace iron

#ifdef SSD_TC_TRACE
extern "C" void iron_ssd_trace(long long* host) { cudaMemcpyFromSymbol(host, iron::g_ssd_trace, sizeof(iron::g_ssd_trace)); }
#endif
