// bf16 GEMM on the 5th-generation tensor cores: C = epilogue(A @ B), f32 accumulation.
//
// Persistent, warp-specialised, one CTA per SM:
//   warp 0      TMA producer: A (128 x 64) and B (BN x 64) tiles, 128-byte swizzle,
//               into a ring of shared-memory stages (mbarrier full/empty pairs)
//   warp 1      MMA issuer: one elected lane issues tcgen05.mma (M 128, N BN, K 16) on
//               shared-memory descriptors, accumulating in tensor memory; tcgen05.commit
//               releases each stage and signals the finished accumulator
//   warps 2..5  epilogue: tcgen05.ld the accumulator (one TMEM lane = one output row per
//               thread), round to bf16, apply the fused output stage, store
// Two accumulators (2 x BN of the 512 TMEM columns) let the MMA warp start the next tile
// while the epilogue drains the previous one.  Tiles are walked M-fastest so the CTAs
// running together share one B (weight) tile through L2.
//
// Every wait on an mbarrier is bounded by a wall-clock limit; a wait that gives up sets
// an abort flag that unwinds all three roles, the producer drains its in-flight copies,
// tensor memory is freed, and the host finds IRON_ERR_TIMEOUT in the status word.
// No multicast: every CTA loads its own operands.
//
// Skinny problems (a decode batch: few rows, so few output tiles) are split along K over
// a thread-block cluster of 2 or 4 CTAs instead: every CTA of a cluster accumulates one
// slice of K for the same tile, the others ship their f32 accumulators into the leader's
// shared memory over distributed shared memory, and after one cluster barrier the leader
// adds them in rank order and runs the output stage.  The result does not depend on timing.
#include <cooperative_groups.h>
#include <cstdlib>
#include <cuda.h>

#include "common.cuh"
#include "tc.cuh"

namespace cg = cooperative_groups;

namespace iron {

constexpr int BM = 128;
constexpr int BK = 64;  // 64 bf16 = 128 bytes: one swizzle-atom row
constexpr int UK = 16;  // K of one tcgen05.mma for 16-bit operands
constexpr int kGemmThreads = 192;

enum { EPI_NONE = 0, EPI_GELU = 1, EPI_SILU = 2, EPI_SIGMOID = 3 };

struct GemmParams {
  void* C;
  const __nv_bfloat16* residual;
  int M, N, K;          // K already bounded by the caller (tensor maps zero-fill past it)
  int ldc;              // elements between rows of C (or between columns when transposed)
  int valid;            // rows of A / C computed
  const int* d_valid;
  int epilogue;
  int out_f32;
  int c_transposed;     // C is (N, M)
  int b_n_major;        // B is (K, N) row-major
  int dual;             // two (N, K) weight matrices: C = bf16(silu(bf16(A W1^T))) * bf16(A W2^T)
  int* status;          // optional device word: receives IRON_ERR_TIMEOUT
  // The fused q/k/v projection of a prompt chunk (pair form only): RoPE in the output stage,
  // q to C, k and v straight into the caches at row rope_start + row.
  const __nv_bfloat16* rope_angles;
  __nv_bfloat16* rope_k;
  __nv_bfloat16* rope_v;
  int rope_H, rope_G, rope_D, rope_start, rope_angle_start;
};

// Instruction descriptor for kind::f16: bf16 x bf16 -> f32, A K-major.
__host__ __device__ constexpr uint32_t make_idesc(int n, bool b_n_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((b_n_major ? 1u : 0u) << 16) |
         ((uint32_t)(n >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
}

constexpr int kMaxSplit = 4;   // CTAs of a cluster that share one tile along K

template <int BN, bool SPLIT = false>
struct GemmCfg {
  static constexpr int kABytes = BM * BK * 2;
  static constexpr int kBBytes = BN * BK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  // The split (skinny) form keeps its footprint to half an SM -- four stages, one 64-column
  // accumulator -- so that the next kernel of a chain can start under it.
  static constexpr int kStages = BN == 256 ? 4 : (BN == 128 ? 6 : 8);
  static constexpr int kTmemCols = SPLIT ? 64 : 512;
  // The leader's landing area for the other CTAs' accumulators lies over the pipeline
  // stages: nothing is shipped before every CTA of the cluster has finished its main loop.
  static constexpr int kStagingBytes = SPLIT ? (kMaxSplit - 1) * BM * BN * 4 : 0;
  static_assert(kStagingBytes <= kStages * kStageBytes, "the staging area must fit in the stages");
  static constexpr int kBarBytes = 256;
  static constexpr int kSmem = kStages * kStageBytes + kBarBytes + 1024;  // + alignment slack
};

__device__ __forceinline__ float epilogue_apply(int mode, float c) {
  // c is already rounded to bf16; the activation's sigmoid is rounded to bf16 before
  // the product, as the reference's output stage does.
  switch (mode) {
    case EPI_GELU: return __fmul_rn(c, 1.0f / (1.0f + expf(-__fmul_rn(1.702f, c))));
    case EPI_SILU: return __fmul_rn(c, round_bf16(1.0f / (1.0f + expf(-c))));
    case EPI_SIGMOID: return 1.0f / (1.0f + expf(-c));
    default: return c;
  }
}

// The output stage for 32 consecutive columns of one row: round, activation, residual,
// store (bf16 or f32; C row-major or transposed).
template <bool kSlim = false>
__device__ __forceinline__ void output_chunk(const GemmParams& p, float* v, int row, int col0) {
  const bool out_f32 = kSlim ? false : p.out_f32 != 0, c_transposed = kSlim ? false : p.c_transposed != 0;
  const int epilogue = kSlim ? EPI_NONE : p.epilogue;
  if (!out_f32) {
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] = epilogue_apply(epilogue, round_bf16(v[j]));
  }
  const bool full_chunk = col0 + 32 <= p.N;
  if (!c_transposed) {
    const size_t off = (size_t)row * p.ldc + col0;
    if (p.residual) {
      // 16-byte loads need every row of the residual to start on an 8-element boundary
      if (full_chunk && (p.ldc & 7) == 0) {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          float f[8];
          unpack8(ld_cached(p.residual + off + q * 8), f);
#pragma unroll
          for (int j = 0; j < 8; ++j) v[q * 8 + j] = __fadd_rn(round_bf16(v[q * 8 + j]), f[j]);
        }
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j)   // unrolled with a predicate: v stays in registers
          if (col0 + j < p.N) v[j] = __fadd_rn(round_bf16(v[j]), __bfloat162float(p.residual[off + j]));
      }
    }
    if (out_f32) {
      float* dst = reinterpret_cast<float*>(p.C) + off;
      if (full_chunk && (p.ldc & 3) == 0) {
#pragma unroll
        for (int q = 0; q < 8; ++q)
          reinterpret_cast<float4*>(dst)[q] = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (col0 + j < p.N) dst[j] = v[j];
      }
    } else {
      __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.C) + off;
      if (full_chunk && (p.ldc & 7) == 0) {
#pragma unroll
        for (int q = 0; q < 4; ++q) reinterpret_cast<uint4*>(dst)[q] = pack8(v + q * 8);
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (col0 + j < p.N) dst[j] = __float2bfloat16_rn(v[j]);
      }
    }
  } else {
    // C is (N, M): lanes hold consecutive rows, so each column is a coalesced run.
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      if (col0 + j >= p.N) break;
      const size_t off = (size_t)(col0 + j) * p.ldc + row;
      float x = v[j];
      if (p.residual) x = __fadd_rn(round_bf16(x), __bfloat162float(p.residual[off]));
      if (out_f32) reinterpret_cast<float*>(p.C)[off] = x;
      else reinterpret_cast<__nv_bfloat16*>(p.C)[off] = __float2bfloat16_rn(x);
    }
  }
}

// kSlim: as for the pair kernel below, the plain product as an instantiation of its own.
template <int BN, bool SPLIT, bool kSlim = false>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                 const __grid_constant__ CUtensorMap map_b2, const GemmParams p) {
  using Cfg = GemmCfg<BN, SPLIT>;
  const int dual = kSlim ? 0 : p.dual;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  float* staging = reinterpret_cast<float*>(smem);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::kStages * Cfg::kStageBytes);
  uint64_t* full = bars;                         // [kStages]
  uint64_t* empty = bars + Cfg::kStages;         // [kStages]
  uint64_t* acc_full = bars + 2 * Cfg::kStages;  // [2]
  uint64_t* acc_empty = acc_full + 2;            // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::kStages; ++s) { mbar_init(full + s, 1); mbar_init(empty + s, 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(acc_full + a, 1); mbar_init(acc_empty + a, 128); }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_b) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_b2) : "memory");
  }
  if (warp == 1) {  // the MMA warp owns tensor memory (all 512 columns unless split)
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"(Cfg::kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // Which tiles and which K blocks this CTA takes: every tile and all of K, or -- split --
  // the cluster's one tile and this rank's slice of K.
  int valid = 0, m_tiles = 0, n_tiles = 0, total = 0, t_first = blockIdx.x, t_step = gridDim.x, k_lo = 0, k_hi = 0;
  unsigned int crank = 0, csize = 1;
  // Output columns per tile: in the gated form one accumulator holds BN/2 columns of the
  // first product and the matching BN/2 columns of the second.
  const int BNO = dual ? BN / 2 : BN;
  const int num_kb = (p.K + BK - 1) / BK;
  auto setup = [&](int rows) {
    valid = max(rows, 0);
    m_tiles = (valid + BM - 1) / BM;
    n_tiles = (p.N + BNO - 1) / BNO;
    total = m_tiles * n_tiles;
    k_hi = num_kb;
    if constexpr (SPLIT) {
      cg::cluster_group cl = cg::this_cluster();
      crank = cl.block_rank();
      csize = cl.num_blocks();
      t_first = blockIdx.x / csize;
      t_step = total > 0 ? total : 1;
      const int per = (num_kb + (int)csize - 1) / (int)csize;
      k_lo = min(num_kb, (int)crank * per);
      k_hi = min(num_kb, k_lo + per);
    }
  };
  // The dependents of this kernel may start their own prologue (and weight loads) now.
  pdl_launch();
  // With the row count known at launch, the weight tiles do not depend on the kernel before:
  // the first stages' B copies go out ahead of the dependency wait.
  const bool early = p.d_valid == nullptr && !p.b_n_major;
  int pre = 0;
  if (early) {
    setup(p.valid);
    if (warp == 0 && lane == 0 && t_first < total) {
      const int n0 = (t_first / m_tiles) * BNO;
      for (int kb = k_lo; kb < k_hi && pre < Cfg::kStages; ++kb, ++pre) {
        mbar_expect_tx(full + pre, Cfg::kStageBytes);
        uint8_t* b_dst = smem + pre * Cfg::kStageBytes + Cfg::kABytes;
        tma_load_2d(b_dst, &map_b, kb * BK, n0, full + pre);
        if (dual) tma_load_2d(b_dst + (BN / 2) * BK * 2, &map_b2, kb * BK, n0, full + pre);
      }
    }
  }
  // A and (for b_n_major) B are inputs the previous kernel may have produced.
  pdl_wait();
  if (!early) setup(p.d_valid ? min(*p.d_valid, p.M) : p.valid);

  if (warp == 0) {
    // ---------------- producer ----------------
    if (lane == 0) {
      int s = 0;
      uint32_t phase = 0;
      int issued = 0;
      bool ok = true;
      for (int t = t_first; t < total && ok; t += t_step) {
        const int m0 = (t % m_tiles) * BM, n0 = (t / m_tiles) * BNO;
        for (int kb = k_lo; kb < k_hi; ++kb) {
          if (!mbar_wait(empty + s, phase ^ 1, abort_flag)) { ok = false; break; }
          uint8_t* a_dst = smem + s * Cfg::kStageBytes;
          uint8_t* b_dst = a_dst + Cfg::kABytes;
          if (issued < pre) {   // this stage's B tile is already on its way
            tma_load_2d(a_dst, &map_a, kb * BK, m0, full + s);
            ++issued;
            if (++s == Cfg::kStages) { s = 0; phase ^= 1; }
            continue;
          }
          mbar_expect_tx(full + s, Cfg::kStageBytes);
          tma_load_2d(a_dst, &map_a, kb * BK, m0, full + s);
          if (dual) {
            tma_load_2d(b_dst, &map_b, kb * BK, n0, full + s);
            tma_load_2d(b_dst + (BN / 2) * BK * 2, &map_b2, kb * BK, n0, full + s);
          } else if (!p.b_n_major) {
            tma_load_2d(b_dst, &map_b, kb * BK, n0, full + s);
          } else {
#pragma unroll
            for (int c = 0; c < BN / 64; ++c)
              tma_load_2d(b_dst + c * (64 * BK * 2), &map_b, n0 + c * 64, kb * BK, full + s);
          }
          ++issued;
          if (++s == Cfg::kStages) { s = 0; phase ^= 1; }
        }
      }
      if (!ok) {
        // Unwinding: let every copy already issued land before the CTA leaves.
        const int outstanding = min(issued, Cfg::kStages);
        int ss = s;
        uint32_t ph = phase;
        for (int i = 0; i < outstanding; ++i) {
          if (--ss < 0) { ss = Cfg::kStages - 1; ph ^= 1; }
          const unsigned long long t0 = global_ns();
          while (!mbar_try_wait(full + ss, ph) && global_ns() - t0 < kWaitLimitNs) {}
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      const uint32_t idesc = make_idesc(BN, p.b_n_major != 0);
      int s = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      for (int t = t_first; t < total && ok; t += t_step, ++it) {
        const int acc = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        if (!mbar_wait(acc_empty + acc, acc_phase ^ 1, abort_flag)) { ok = false; break; }
        tcgen05_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = k_lo; kb < k_hi; ++kb) {
          if (!mbar_wait(full + s, phase, abort_flag)) { ok = false; break; }
          tcgen05_fence_after();
          const uint32_t a_addr = smem_u32(smem + s * Cfg::kStageBytes);
          const uint32_t b_addr = a_addr + Cfg::kABytes;
#pragma unroll
          for (int k = 0; k < BK / UK; ++k) {
            // K-major: 128-byte rows, 8-row groups 1024 bytes apart, 32 bytes per K step.
            const uint64_t a_desc = make_desc(a_addr + k * UK * 2, 16, 1024);
            // N-major B: 64-column chunks 8 KB apart, 8-row K groups 1024 bytes apart,
            // one K step is 16 rows of 128 bytes.
            const uint64_t b_desc = p.b_n_major ? make_desc(b_addr + k * UK * 128, 64 * BK * 2, 1024)
                                                : make_desc(b_addr + k * UK * 2, 16, 1024);
            tcgen05_mma_bf16(d_tmem, a_desc, b_desc, idesc, kb != k_lo || k != 0);
          }
          tcgen05_commit(empty + s);  // the stage is free once these MMAs have read it
          if (++s == Cfg::kStages) { s = 0; phase ^= 1; }
        }
        if (ok) tcgen05_commit(acc_full + acc);
      }
    }
  }
  // ---------------- epilogue (warps 2..5) ----------------
  // `ship`: this CTA's accumulator goes to the cluster leader's staging area as it is;
  // `gather`: the other ranks' accumulators are added to this one before the output stage.
  auto drain = [&](bool ship, bool gather) {
    const int group = warp & 3;  // the TMEM lane quarter this warp may read
    int it = 0;
    bool ok = true;
    for (int t = t_first; t < total && ok; t += t_step, ++it) {
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      const int m0 = (t % m_tiles) * BM, n0 = (t / m_tiles) * BNO;
      if (!mbar_wait(acc_full + acc, acc_phase, abort_flag)) { ok = false; break; }
      tcgen05_fence_after();
      const int row = m0 + group * 32 + lane;
      const bool row_live = row < valid;
#pragma unroll 1
      for (int c = 0; c < BNO / 32; ++c) {
        uint32_t r[32];
        tmem_ld32(tmem_base + ((uint32_t)(group * 32) << 16) + acc * BN + c * 32, r);
        tmem_ld_wait();
        const int col0 = n0 + c * 32;
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
        if (dual) {
          // the second product's columns sit BN/2 further in the accumulator
          tmem_ld32(tmem_base + ((uint32_t)(group * 32) << 16) + acc * BN + BN / 2 + c * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j)
            v[j] = __fmul_rn(round_bf16(silu_f32(round_bf16(v[j]))), round_bf16(__uint_as_float(r[j])));
        }
        if (!row_live || col0 >= p.N) continue;
        if constexpr (SPLIT) {
          const size_t mine = ((size_t)(group * 32 + lane)) * BN + c * 32;
          if (ship) {
            float* dst = cg::this_cluster().map_shared_rank(staging, 0) + (size_t)(crank - 1) * BM * BN + mine;
#pragma unroll
            for (int q = 0; q < 8; ++q)
              reinterpret_cast<float4*>(dst)[q] = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
            continue;
          }
          if (gather) {
            for (unsigned int rk = 1; rk < csize; ++rk) {
              const float4* src = reinterpret_cast<const float4*>(staging + (size_t)(rk - 1) * BM * BN + mine);
#pragma unroll
              for (int q = 0; q < 8; ++q) {
                const float4 f = src[q];
                v[4 * q] += f.x; v[4 * q + 1] += f.y; v[4 * q + 2] += f.z; v[4 * q + 3] += f.w;
              }
            }
          }
        }
        output_chunk<kSlim>(p, v, row, col0);
      }
      tcgen05_fence_before();
      mbar_arrive(acc_empty + acc);
    }
  };
  if constexpr (!SPLIT) {
    if (warp >= 2) drain(false, false);
  } else {
    // every CTA's main loop is over (its copies have landed and its MMAs have read them)
    // before anything is written over the leader's stages
    if (warp >= 2 && t_first < total) mbar_wait(acc_full, 0, abort_flag);
    cg::this_cluster().sync();
    if (warp >= 2 && crank != 0) drain(true, false);
    cg::this_cluster().sync();   // every rank's accumulator is in the leader's staging area
    if (warp >= 2 && crank == 0) drain(false, true);
  }

  tcgen05_fence_before();
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag && p.status) *p.status = IRON_ERR_TIMEOUT;
  if (warp == 1) {
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(Cfg::kTmemCols)
                 : "memory");
  }
}


// ---- the CTA-pair form ---------------------------------------------------------------
// Two CTAs of a cluster, on two SMs, compute one 256 x 256 tile with tcgen05.mma
// cta_group::2: each CTA stages its own 128 rows of A and its own half (128 of the 256
// columns) of B, the leader's MMA warp issues one instruction that reads both CTAs'
// shared memory, and each CTA's tensor memory receives the accumulator of its 128 rows.
// Per SM and K block that is 32 KB of operands from L2 for the same math as the 48 KB of
// the one-CTA form: the main loop is bound by L2 -> SM bandwidth, so this is what moves it.
//
// Protocol (every barrier wait bounded, as above):
//   full[s]      in the leader; the leader's producer arms it with both CTAs' bytes and
//                both producers' TMA copies complete on it (cta_group::2 lets a copy
//                signal the peer's barrier).  No copy is multicast.
//   empty[s]     in both CTAs; the leader's tcgen05.commit arrives on both.
//   acc_full[a]  in both CTAs; the same.
//   acc_empty[a] in the leader, 256 arrivals: both CTAs' epilogue threads.
// In the gated form the leader stages the first weight matrix's rows and the peer the
// second's, so accumulator columns 0..127 / 128..255 hold the two products as in the
// one-CTA gated form.
constexpr int kPairStages = 6;
constexpr int kPairAccStride = 256;                // tensor-memory columns between the two accumulators
constexpr int kPairABytes = BM * BK * 2;           // this CTA's 128 rows of A
// PBN: columns of a pair's tile, 256 or 192 (the narrower tile when it saves a wave of tiles).
template <int PBN>
struct PairCfg {
  static constexpr int kBBytes = (PBN / 2) * BK * 2;   // this CTA's half of the tile's columns of B
  static constexpr int kStageBytes = kPairABytes + kBBytes;
  static constexpr int kSmem = kPairStages * kStageBytes + 256 + 1024;
};

__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// The shared::cluster address of the same shared-memory offset in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t map_to_rank(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, int x, int y, uint32_t bar_cluster) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(x), "r"(y), "r"(bar_cluster)
      : "memory");
}
__device__ __forceinline__ void tcgen05_commit_pair(uint64_t* bar) {
  // arrives on the barrier at this offset in both CTAs of the pair
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(smem_u32(bar)), "h"((uint16_t)3)
               : "memory");
}
__device__ __forceinline__ void tcgen05_mma_bf16_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                                      uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// kSlim: the plain product (bf16 row-major C, optional residual, no activation, no gated pair, no RoPE) as an
// instantiation of its own: the other output stages are compiled out of it.
template <int PBN, bool kSlim = false>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kGemmThreads, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                 const __grid_constant__ CUtensorMap map_b2, const GemmParams p) {
  constexpr int kPairBN = PBN;
  const int dual = kSlim ? 0 : p.dual;
  const __nv_bfloat16* const rope_angles = kSlim ? nullptr : p.rope_angles;
  constexpr int kPairStageBytes = PairCfg<PBN>::kStageBytes;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kPairStages * kPairStageBytes);
  uint64_t* full = bars;                        // [kPairStages], used in the leader
  uint64_t* empty = bars + kPairStages;         // [kPairStages]
  uint64_t* acc_full = bars + 2 * kPairStages;  // [2]
  uint64_t* acc_empty = acc_full + 2;           // [2], used in the leader
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_rank();   // 0: the leader
  const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kPairStages; ++s) { mbar_init(full + s, 1); mbar_init(empty + s, 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(acc_full + a, 1); mbar_init(acc_empty + a, 256); }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_b) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_b2) : "memory");
  }
  if (warp == 1) {  // each CTA's MMA warp takes part in the pair's allocation (all 512 columns)
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"(512)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tcgen05_fence_before();
  __syncthreads();
  cluster_sync_all();   // both CTAs' barriers are initialised before either is signalled
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int BNO = dual ? kPairBN / 2 : kPairBN;
  const int num_kb = (p.K + BK - 1) / BK;
  pdl_launch();
  // With the row count known at launch, the first tile's weight (B) copies do not depend on the
  // kernel before: they go out ahead of the dependency wait, one per pipeline stage.
  int pre = 0;
  if (p.d_valid == nullptr && warp == 0 && lane == 0) {
    const int v0 = max(p.valid, 0), mt = (v0 + 2 * BM - 1) / (2 * BM);
    if (mt > 0 && pair < mt * ((p.N + BNO - 1) / BNO)) {
      const int n0 = (pair / mt) * BNO;
      for (int kb = 0; kb < num_kb && pre < kPairStages; ++kb, ++pre) {
        uint8_t* b_dst = smem + pre * kPairStageBytes + kPairABytes;
        const uint32_t bar = map_to_rank(smem_u32(full + pre), 0);
        if (rank == 0) mbar_expect_tx(full + pre, 2 * kPairStageBytes);
        if (dual) tma_load_2d_pair(b_dst, rank == 0 ? &map_b : &map_b2, kb * BK, n0, bar);
        else tma_load_2d_pair(b_dst, &map_b, kb * BK, n0 + (int)rank * (kPairBN / 2), bar);
      }
    }
  }
  pdl_wait();   // A, and the residual, are the previous kernels' outputs
  const int valid = max(p.d_valid ? min(*p.d_valid, p.M) : p.valid, 0);
  const int m_tiles = (valid + 2 * BM - 1) / (2 * BM);
  const int n_tiles = (p.N + BNO - 1) / BNO;
  const int total = m_tiles * n_tiles;

  if (warp == 0) {
    // ---------------- producer (one per CTA) ----------------
    if (lane == 0) {
      int s = 0, issued = pre > 0 ? 1 : 0;
      int early = pre;   // stages whose B copy is already on its way
      uint32_t phase = 0;
      bool ok = true;
      for (int t = pair; t < total && ok; t += pairs) {
        const int m0 = (t % m_tiles) * (2 * BM) + (int)rank * BM;
        const int n0 = (t / m_tiles) * BNO;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(empty + s, phase ^ 1, abort_flag)) { ok = false; break; }
          uint8_t* a_dst = smem + s * kPairStageBytes;
          uint8_t* b_dst = a_dst + kPairABytes;
          const uint32_t bar = map_to_rank(smem_u32(full + s), 0);
          if (early > 0) {
            --early;
            tma_load_2d_pair(a_dst, &map_a, kb * BK, m0, bar);
            ++issued;
            if (++s == kPairStages) { s = 0; phase ^= 1; }
            continue;
          }
          if (rank == 0) mbar_expect_tx(full + s, 2 * kPairStageBytes);
          tma_load_2d_pair(a_dst, &map_a, kb * BK, m0, bar);
          if (dual) tma_load_2d_pair(b_dst, rank == 0 ? &map_b : &map_b2, kb * BK, n0, bar);
          else tma_load_2d_pair(b_dst, &map_b, kb * BK, n0 + (int)rank * (kPairBN / 2), bar);
          ++issued;
          if (++s == kPairStages) { s = 0; phase ^= 1; }
        }
      }
      if (!ok) {
        // Unwinding: this CTA's copies land in its own shared memory but complete on the
        // leader's barrier, which the peer cannot poll: give them a millisecond, many
        // times what a copy takes, before the CTA may leave.
        if (issued > 0) {
          const unsigned long long t0 = global_ns();
          while (global_ns() - t0 < 1000000ull) {}
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (the leader's) ----------------
    if (rank == 0) {
      // The whole warp runs the loop and one elected lane issues (see elect_one); every lane
      // probes the barriers, and the outcome is made uniform before anyone leaves the loop.
      // M 256 across the pair (128 rows per CTA), N 256
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(kPairBN >> 3) << 17) |
                             ((uint32_t)((2 * BM) >> 4) << 24);
      int s = 0, it = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = pair; t < total && ok; t += pairs, ++it) {
        const int acc = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        ok = __all_sync(0xffffffffu, mbar_wait(acc_empty + acc, acc_phase ^ 1, abort_flag));
        if (!ok) break;
        tcgen05_fence_after();
        const uint32_t d_tmem = tmem_base + acc * kPairAccStride;
        for (int kb = 0; kb < num_kb; ++kb) {
          ok = __all_sync(0xffffffffu, mbar_wait(full + s, phase, abort_flag));
          if (!ok) break;
          tcgen05_fence_after();
          const uint32_t a_addr = smem_u32(smem + s * kPairStageBytes);
          const uint32_t b_addr = a_addr + kPairABytes;
          if (elect_one()) {
#pragma unroll
            for (int k = 0; k < BK / UK; ++k) {
              const uint64_t a_desc = make_desc(a_addr + k * UK * 2, 16, 1024);
              const uint64_t b_desc = make_desc(b_addr + k * UK * 2, 16, 1024);
              tcgen05_mma_bf16_pair(d_tmem, a_desc, b_desc, idesc, kb != 0 || k != 0);
            }
            tcgen05_commit_pair(empty + s);
          }
          __syncwarp();
          if (++s == kPairStages) { s = 0; phase ^= 1; }
        }
        if (ok && elect_one()) tcgen05_commit_pair(acc_full + acc);
        __syncwarp();
      }
    }
  } else {
    // ---------------- epilogue (warps 2..5 of each CTA: its own 128 rows) ----------------
    const int group = warp & 3;
    int it = 0;
    bool ok = true;
    for (int t = pair; t < total && ok; t += pairs, ++it) {
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      const int m0 = (t % m_tiles) * (2 * BM) + (int)rank * BM, n0 = (t / m_tiles) * BNO;
      if (!mbar_wait(acc_full + acc, acc_phase, abort_flag)) { ok = false; break; }
      tcgen05_fence_after();
      const int row = m0 + group * 32 + lane;
      const bool row_live = row < valid;
      if (rope_angles) {
        // A tile holds whole heads (BNO % D == 0).  Per head and per run of 32 rotation pairs:
        // element i and element i + D/2, rounded to bf16 as the projection's output is, then
        // turned with the products and the sum each rounded once -- the arithmetic of the
        // separate RoPE kernel -- and stored where that kernel stores them.
        const int D = p.rope_D, half = D >> 1, H = p.rope_H, G = p.rope_G;
        const uint32_t t_row = tmem_base + ((uint32_t)(group * 32) << 16) + acc * kPairAccStride;
#pragma unroll 1
        for (int hl = 0; hl < BNO / D; ++hl) {
          const int hh = n0 / D + hl;
          if (hh >= H + 2 * G) break;
#pragma unroll 1
          for (int s = 0; s < half / 32; ++s) {
            uint32_t ra[32], rb[32];
            tmem_ld32(t_row + hl * D + s * 32, ra);
            tmem_ld32(t_row + hl * D + half + s * 32, rb);
            tmem_ld_wait();
            if (!row_live) continue;
            float a[32], b[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              a[j] = round_bf16(__uint_as_float(ra[j]));
              b[j] = round_bf16(__uint_as_float(rb[j]));
            }
            if (hh < H + G) {
              const __nv_bfloat16* ar = rope_angles + (size_t)(p.rope_angle_start + row) * D + 2 * (s * 32);
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                float cs[16];
                unpack8(ld_cached(ar + q * 16), cs);
                unpack8(ld_cached(ar + q * 16 + 8), cs + 8);
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                  const float c = cs[2 * j], sn = cs[2 * j + 1];
                  const float x = a[q * 8 + j], y = b[q * 8 + j];
                  a[q * 8 + j] = __fsub_rn(__fmul_rn(x, c), __fmul_rn(y, sn));
                  b[q * 8 + j] = __fadd_rn(__fmul_rn(y, c), __fmul_rn(x, sn));
                }
              }
            }
            __nv_bfloat16* dst;
            if (hh < H) dst = reinterpret_cast<__nv_bfloat16*>(p.C) + (size_t)row * p.ldc + (size_t)hh * D;
            else if (hh < H + G) dst = p.rope_k + ((size_t)(p.rope_start + row) * G + (hh - H)) * D;
            else dst = p.rope_v + ((size_t)(p.rope_start + row) * G + (hh - H - G)) * D;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              reinterpret_cast<uint4*>(dst + s * 32)[q] = pack8(a + q * 8);
              reinterpret_cast<uint4*>(dst + half + s * 32)[q] = pack8(b + q * 8);
            }
          }
        }
        tcgen05_fence_before();
        mbar_arrive_cluster(map_to_rank(smem_u32(acc_empty + acc), 0));
        continue;
      }
#pragma unroll 1
      for (int c = 0; c < BNO / 32; ++c) {
        uint32_t r[32];
        tmem_ld32(tmem_base + ((uint32_t)(group * 32) << 16) + acc * kPairAccStride + c * 32, r);
        tmem_ld_wait();
        const int col0 = n0 + c * 32;
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
        if (dual) {
          tmem_ld32(tmem_base + ((uint32_t)(group * 32) << 16) + acc * kPairAccStride + kPairBN / 2 + c * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j)
            v[j] = __fmul_rn(round_bf16(silu_f32(round_bf16(v[j]))), round_bf16(__uint_as_float(r[j])));
        }
        if (!row_live || col0 >= p.N) continue;
        output_chunk<kSlim>(p, v, row, col0);
      }
      tcgen05_fence_before();
      mbar_arrive_cluster(map_to_rank(smem_u32(acc_empty + acc), 0));
    }
  }

  tcgen05_fence_before();
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag && p.status) *p.status = IRON_ERR_TIMEOUT;
  // neither CTA leaves, or frees the pair's tensor memory, while the other may still signal
  // its barriers or read its shared memory
  cluster_sync_all();
  if (warp == 1) {
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
  }
}

// ---- host side ---------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
  }
  return fn;
}

// The weight-streaming form for a decode batch (gemm_skinny.cu).
int launch_gemm_skinny(const void* X, const void* W, const void* W2, void* C, const void* residual, int rows, int N,
                       int K, int ldx, int ldw, int ldc, int* d_status, cudaStream_t stream);

// A 2-D bf16 tensor map: `inner` contiguous elements per row, `outer` rows `pitch` elements apart.
static bool make_map(CUtensorMap* map, const void* base, uint64_t inner, uint64_t outer, uint64_t pitch,
                     uint32_t box_inner, uint32_t box_outer) {
  EncodeTiledFn fn = encode_tiled();
  if (!fn) return false;
  const cuuint64_t dims[2] = {inner, outer};
  const cuuint64_t strides[1] = {pitch * 2};
  const cuuint32_t box[2] = {box_inner, box_outer};
  const cuuint32_t elem[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int BN>
static int launch_gemm(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mb2, const GemmParams& p,
                       int max_rows, cudaStream_t stream) {
  using Cfg = GemmCfg<BN>;
  static DeviceOnce configured;   // the attribute is per device
  if (!configured.done()) {
    if (cudaFuncSetAttribute(gemm_bf16_kernel<BN, false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             Cfg::kSmem) != cudaSuccess ||
        cudaFuncSetAttribute(gemm_bf16_kernel<BN, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             Cfg::kSmem) != cudaSuccess)
      return IRON_ERR_LAUNCH;
    configured.mark();
  }
  const int bno = p.dual ? BN / 2 : BN;
  const int tiles = ((max_rows + BM - 1) / BM) * ((p.N + bno - 1) / bno);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(tiles < kSMs ? (tiles < 1 ? 1 : tiles) : kSMs);
  cfg.blockDim = dim3(kGemmThreads);
  cfg.dynamicSmemBytes = Cfg::kSmem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  fill_pdl_attr(cfg, attr);
  static const bool slim_on = [] { const char* e = getenv("IRON_GEMM_SLIM"); return !(e && e[0] == '0'); }();
  const bool slim = slim_on && !p.dual && !p.out_f32 && !p.c_transposed && p.epilogue == EPI_NONE;
  const cudaError_t e = slim ? cudaLaunchKernelEx(&cfg, gemm_bf16_kernel<BN, false, true>, ma, mb, mb2, p)
                             : cudaLaunchKernelEx(&cfg, gemm_bf16_kernel<BN, false, false>, ma, mb, mb2, p);
  return e == cudaSuccess ? IRON_OK : IRON_ERR_LAUNCH;
}

// One tile per cluster of `splits` CTAs, each taking a slice of K.
static int launch_gemm_split(const CUtensorMap& ma, const CUtensorMap& mb, const GemmParams& p, int tiles,
                             int splits, cudaStream_t stream) {
  using Cfg = GemmCfg<64, true>;
  static DeviceOnce configured;   // the attribute is per device
  if (!configured.done()) {
    if (cudaFuncSetAttribute(gemm_bf16_kernel<64, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             Cfg::kSmem) != cudaSuccess)
      return IRON_ERR_LAUNCH;
    configured.mark();
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(tiles * splits);
  cfg.blockDim = dim3(kGemmThreads);
  cfg.dynamicSmemBytes = Cfg::kSmem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = splits;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1 + pdl_attr_count();
  return cudaLaunchKernelEx(&cfg, gemm_bf16_kernel<64, true>, ma, mb, mb, p) == cudaSuccess ? IRON_OK
                                                                                            : IRON_ERR_LAUNCH;
}

// One 256 x 256 tile per CTA pair; pairs walk the tiles M-fastest.
template <int PBN>
static int launch_gemm_pair(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mb2,
                            const GemmParams& p, int max_rows, cudaStream_t stream) {
  constexpr int kPairBN = PBN;
  constexpr int kPairSmem = PairCfg<PBN>::kSmem;
  static DeviceOnce configured;   // the attribute is per device
  if (!configured.done()) {
    if (cudaFuncSetAttribute(gemm_pair_kernel<PBN, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kPairSmem) !=
            cudaSuccess ||
        cudaFuncSetAttribute(gemm_pair_kernel<PBN, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kPairSmem) !=
            cudaSuccess)
      return IRON_ERR_LAUNCH;
    configured.mark();
  }
  const int bno = p.dual ? kPairBN / 2 : kPairBN;
  const int tiles = ((max_rows + 2 * BM - 1) / (2 * BM)) * ((p.N + bno - 1) / bno);
  const int pairs = tiles < kSMs / 2 ? (tiles < 1 ? 1 : tiles) : kSMs / 2;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * pairs);
  cfg.blockDim = dim3(kGemmThreads);
  cfg.dynamicSmemBytes = kPairSmem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  fill_pdl_attr(cfg, attr);
  static const bool slim_on = [] { const char* e = getenv("IRON_GEMM_SLIM"); return !(e && e[0] == '0'); }();
  const bool slim = slim_on && !p.dual && !p.rope_angles && !p.out_f32 && !p.c_transposed && p.epilogue == EPI_NONE;
  const cudaError_t e = slim ? cudaLaunchKernelEx(&cfg, gemm_pair_kernel<PBN, true>, ma, mb, mb2, p)
                             : cudaLaunchKernelEx(&cfg, gemm_pair_kernel<PBN, false>, ma, mb, mb2, p);
  return e == cudaSuccess ? IRON_OK : IRON_ERR_LAUNCH;
}

// The pair form takes K-major B (weights as stored) and problems with more than one
// 128-row tile of A; IRON_GEMM_PAIR=0 keeps every problem on the one-CTA form.
static bool pair_enabled() {
  static int on = -1;
  if (on < 0) {
    const char* e = getenv("IRON_GEMM_PAIR");
    on = (e && e[0] == '0') ? 0 : 1;
  }
  return on != 0;
}

}  // namespace iron

using namespace iron;

extern "C" int iron_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb,
                              int ldc, int b_col_maj, int c_col_maj, int valid_rows, const int* d_valid_rows,
                              int valid_k, int epilogue, const void* residual, int out_f32, int* d_status,
                              iron_stream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return IRON_ERR_SHAPE;
  if (valid_rows < 0 || valid_rows > M || valid_k < 0 || valid_k > K) return IRON_ERR_SHAPE;
  if (epilogue < EPI_NONE || epilogue > EPI_SIGMOID) return IRON_ERR_SHAPE;
  if (out_f32 && epilogue != EPI_NONE) return IRON_ERR_UNSUPPORTED;
  // TMA: 16-byte aligned bases and row pitches
  if (!aligned16(A) || !aligned16(B) || !aligned16(C)) return IRON_ERR_ALIGN;
  // the residual shares C's pitch; its rows are read 16 bytes at a time when that pitch allows
  if (residual && !aligned16(residual)) return IRON_ERR_ALIGN;
  if ((lda & 7) || (ldb & 7)) return IRON_ERR_ALIGN;
  if (lda < K || ldb < (b_col_maj ? K : N) || ldc < (c_col_maj ? M : N)) return IRON_ERR_SHAPE;
  if (valid_rows == 0 && !d_valid_rows) return IRON_OK;
  if (valid_k == 0) return IRON_ERR_SHAPE;

  // a decode batch against weights as stored: the weight-streaming kernel with the operands swapped
  if (valid_rows >= 1 && valid_rows <= 64 && !d_valid_rows && b_col_maj && !c_col_maj && !out_f32 &&
      epilogue == EPI_NONE && (ldb & 7) == 0) {
    const int rc = launch_gemm_skinny(A, B, nullptr, C, residual, valid_rows, N, valid_k, lda, ldb, ldc, d_status,
                                      (cudaStream_t)stream);
    if (rc != IRON_ERR_UNSUPPORTED) return rc;
  }
  // BN: the widest tile that still yields at least one wave of CTAs
  const int m_tiles = (M + BM - 1) / BM;
  int bn = 256;
  if (N <= 64 || (long long)m_tiles * ((N + 255) / 256) < kSMs / 2) bn = 128;
  if (N <= 64 || (bn == 128 && (long long)m_tiles * ((N + 127) / 128) < kSMs / 2)) bn = 64;

  CUtensorMap ma, mb;
  if (!make_map(&ma, A, (uint64_t)valid_k, (uint64_t)M, (uint64_t)lda, BK, BM)) return IRON_ERR_LAUNCH;
  bool okb;
  if (b_col_maj) okb = make_map(&mb, B, (uint64_t)valid_k, (uint64_t)N, (uint64_t)ldb, BK, bn);
  else okb = make_map(&mb, B, (uint64_t)N, (uint64_t)valid_k, (uint64_t)ldb, 64, BK);
  if (!okb) return IRON_ERR_LAUNCH;

  GemmParams p = {};
  p.C = C; p.residual = (const __nv_bfloat16*)residual;
  p.M = M; p.N = N; p.K = valid_k; p.ldc = ldc;
  p.valid = valid_rows; p.d_valid = d_valid_rows;
  p.epilogue = epilogue; p.out_f32 = out_f32; p.c_transposed = c_col_maj; p.b_n_major = !b_col_maj;
  p.status = d_status;
  const int max_rows = d_valid_rows ? M : valid_rows;
  cudaStream_t s = (cudaStream_t)stream;
  if (bn == 64) {
    // few tiles (a decode batch): split K over a cluster so that more SMs stream the weights
    const int tiles = ((max_rows + BM - 1) / BM) * ((N + 63) / 64);
    const int num_kb = (valid_k + BK - 1) / BK;
    int splits = 1;
    while (splits < kMaxSplit && tiles * splits * 2 <= kSMs && num_kb / (splits * 2) >= 4) splits *= 2;
    if (splits > 1 && tiles >= 1) return launch_gemm_split(ma, mb, p, tiles, splits, s);
  }
  if (bn == 256 && b_col_maj && max_rows > BM && pair_enabled()) {
    // 192-column tiles when they finish in fewer, or shorter, waves over the 74 pairs
    const long long mt2 = (max_rows + 2 * BM - 1) / (2 * BM);
    auto cost = [&](int bn_) { return ((mt2 * ((N + bn_ - 1) / bn_) + kSMs / 2 - 1) / (kSMs / 2)) * bn_; };
    // (the narrower tile re-reads A more often per flop: it must save more than a seventh)
    const int pbn = cost(192) * 8 < cost(256) * 7 ? 192 : 256;
    CUtensorMap mh;   // each CTA of a pair stages half of the tile's rows of B
    if (!make_map(&mh, B, (uint64_t)valid_k, (uint64_t)N, (uint64_t)ldb, BK, pbn / 2)) return IRON_ERR_LAUNCH;
    return pbn == 192 ? launch_gemm_pair<192>(ma, mh, mh, p, max_rows, s)
                      : launch_gemm_pair<256>(ma, mh, mh, p, max_rows, s);
  }
  if (bn == 256) return launch_gemm<256>(ma, mb, mb, p, max_rows, s);
  if (bn == 128) return launch_gemm<128>(ma, mb, mb, p, max_rows, s);
  return launch_gemm<64>(ma, mb, mb, p, max_rows, s);
}

extern "C" int iron_gemm_qkv_rope_bf16(const void* A, const void* Wqkv, void* qkv, int M, int K, int lda, int ldb,
                                       int ldc, int valid_rows, const void* angles, void* k_cache, void* v_cache,
                                       int H, int G, int D, int start, int angle_start, int* d_status,
                                       iron_stream_t stream) {
  if (M <= 0 || K <= 0 || H <= 0 || G <= 0 || (D != 64 && D != 128)) return IRON_ERR_SHAPE;
  if (valid_rows < 0 || valid_rows > M || start < 0 || angle_start < 0) return IRON_ERR_SHAPE;
  const int N = (H + 2 * G) * D;
  if (!aligned16(A) || !aligned16(Wqkv) || !aligned16(qkv) || !aligned16(angles) || !aligned16(k_cache) ||
      !aligned16(v_cache))
    return IRON_ERR_ALIGN;
  if ((lda & 7) || (ldb & 7) || (ldc & 7)) return IRON_ERR_ALIGN;
  if (lda < K || ldb < K || ldc < N) return IRON_ERR_SHAPE;
  // the pair form only, with tiles of whole heads; the caller runs the two kernels otherwise
  if (valid_rows <= BM || !pair_enabled()) return IRON_ERR_UNSUPPORTED;
  const long long mt2 = (valid_rows + 2 * BM - 1) / (2 * BM);
  auto cost = [&](int bn_) { return ((mt2 * ((N + bn_ - 1) / bn_) + kSMs / 2 - 1) / (kSMs / 2)) * bn_; };
  const int pbn = (D == 64 && cost(192) * 8 < cost(256) * 7) ? 192 : 256;
  CUtensorMap ma, mh;
  if (!make_map(&ma, A, (uint64_t)K, (uint64_t)M, (uint64_t)lda, BK, BM) ||
      !make_map(&mh, Wqkv, (uint64_t)K, (uint64_t)N, (uint64_t)ldb, BK, pbn / 2))
    return IRON_ERR_LAUNCH;
  GemmParams p = {};
  p.C = qkv; p.M = M; p.N = N; p.K = K; p.ldc = ldc; p.valid = valid_rows; p.status = d_status;
  p.rope_angles = (const __nv_bfloat16*)angles; p.rope_k = (__nv_bfloat16*)k_cache; p.rope_v = (__nv_bfloat16*)v_cache;
  p.rope_H = H; p.rope_G = G; p.rope_D = D; p.rope_start = start; p.rope_angle_start = angle_start;
  cudaStream_t s = (cudaStream_t)stream;
  return pbn == 192 ? launch_gemm_pair<192>(ma, mh, mh, p, valid_rows, s)
                    : launch_gemm_pair<256>(ma, mh, mh, p, valid_rows, s);
}

extern "C" int iron_gemm_swiglu_bf16(const void* A, const void* Wg, const void* Wu, void* C, int M, int N, int K,
                                     int lda, int ldb, int ldc, int valid_rows, const int* d_valid_rows,
                                     int* d_status, iron_stream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return IRON_ERR_SHAPE;
  if (valid_rows < 0 || valid_rows > M) return IRON_ERR_SHAPE;
  if (!aligned16(A) || !aligned16(Wg) || !aligned16(Wu) || !aligned16(C)) return IRON_ERR_ALIGN;
  if ((lda & 7) || (ldb & 7)) return IRON_ERR_ALIGN;
  if (lda < K || ldb < K || ldc < N) return IRON_ERR_SHAPE;
  if (valid_rows == 0 && !d_valid_rows) return IRON_OK;
  if (valid_rows >= 1 && valid_rows <= 64 && !d_valid_rows) {
    const int rc = launch_gemm_skinny(A, Wg, Wu, C, nullptr, valid_rows, N, K, lda, ldb, ldc, d_status,
                                      (cudaStream_t)stream);
    if (rc != IRON_ERR_UNSUPPORTED) return rc;
  }
  // One 128 x BN accumulator = BN/2 output columns: the gate half and the up half.  The
  // widest tile that still gives at least half a wave of CTAs.
  const int max_rows = d_valid_rows ? M : valid_rows;
  const int m_tiles = (max_rows + BM - 1) / BM;
  int bn = 256;
  if ((long long)m_tiles * ((N + 127) / 128) < kSMs / 2) bn = 128;
  if (bn == 128 && (long long)m_tiles * ((N + 63) / 64) < kSMs / 2) bn = 64;
  CUtensorMap ma, mg, mu;
  if (!make_map(&ma, A, (uint64_t)K, (uint64_t)M, (uint64_t)lda, BK, BM) ||
      !make_map(&mg, Wg, (uint64_t)K, (uint64_t)N, (uint64_t)ldb, BK, bn / 2) ||
      !make_map(&mu, Wu, (uint64_t)K, (uint64_t)N, (uint64_t)ldb, BK, bn / 2))
    return IRON_ERR_LAUNCH;
  GemmParams p = {};
  p.C = C; p.M = M; p.N = N; p.K = K; p.ldc = ldc;
  p.valid = valid_rows; p.d_valid = d_valid_rows;
  p.epilogue = EPI_NONE; p.dual = 1; p.status = d_status;
  cudaStream_t s = (cudaStream_t)stream;
  if (bn == 256 && max_rows > BM && pair_enabled()) return launch_gemm_pair<256>(ma, mg, mu, p, max_rows, s);
  if (bn == 256) return launch_gemm<256>(ma, mg, mu, p, max_rows, s);
  if (bn == 128) return launch_gemm<128>(ma, mg, mu, p, max_rows, s);
  return launch_gemm<64>(ma, mg, mu, p, max_rows, s);
}
