// C = X W^T for a few rows of X (a decode batch: 1 to 64 rows) and a large weight matrix W (N, K):
// the weights cross HBM once and that is the whole cost, so the kernel is built around streaming
// them, with the operands' roles swapped.
//
// iron/operators/gemm.py:143 is the operator; a batched decode step of iron/lm/blocks.py's
// projections (q/k/v, o_proj, gate/up, down_proj, the head) is where it has this shape.
//
// The 128-row tcgen05.mma wants 128 rows of SOMETHING: with X as its A operand more than half of
// every product is padding and each k block moves 16 KB of (mostly zero) X beside 8 KB of
// weights.  Here the WEIGHTS are the A operand -- a tile is 128 weight rows (or, in the gated
// form, 64 rows of the gate matrix and the matching 64 of the up matrix) -- and the batch is
// the 64-column B operand: C^T (128 x 64) accumulates in tensor memory, a k block moves 16 KB
// of weights and 8 KB of X (from L2), and a CTA is a four-stage TMA pipeline (96 KB in flight,
// under half an SM: two kernels of a chain overlap).  Few tiles (q/k/v: 24, o_proj and down_proj: 16) are split along K over a
// cluster of 2, 4 or 8 CTAs so that 100 to 128 SMs stream; each CTA parks its partial tile in
// its own shared memory (over the drained stages) and, after one cluster barrier, reduces ITS eighth (quarter, half) of
// the tile's rows over distributed shared memory in rank order, applies the output stage
// (round; residual; or silu(gate) * up) and writes C.  The first weight tiles are on their way
// before the dependency wait.  Every wait is bounded (2 s -> IRON_ERR_TIMEOUT).
//
// Two neighbours of a projection in a decoder layer fold in (iron/lm/blocks.py: RMSNorm before q/k/v and
// before gate/up; RoPE and the cache write after q/k/v):
//   * RMSNorm.  A projection with a residual (o_proj, down_proj) also leaves, per batch row and per CTA, the
//     sum of squares of the bf16 values it wrote (a fixed slot each: no atomics, the same bits every run).
//     The projection that follows adds the slots in order, and its four output warps -- idle until the
//     last product -- turn each X tile the TMA has landed into bf16(bf16(x / rms) * weight), the RMSNorm
//     kernel's two roundings, in place (128-byte-swizzled as the TMA wrote it) before the products read
//     it.  The normalised activations never exist in HBM and the norm is no launch.
//   * RoPE + cache write.  The q/k/v form reduces PAIRS (i, i + D/2) of a head instead of runs of
//     features, rotates q and k by the angle row of the sequence's position, and writes q densely and
//     k / v into row `position` of that sequence's caches.
#include <cooperative_groups.h>
#include <cuda.h>

#include "tc.cuh"

namespace cg = cooperative_groups;

namespace iron {

constexpr int kSkThreads = 192;        // warp 0 TMA, warp 1 MMA, warps 2-5 output
constexpr int kSkStages = 4;            // when K is split over a cluster (short loops, small footprint)
constexpr int kSkMaxStages = 8;         // one CTA a tile, all of K: a deeper pipeline, the whole SM
constexpr int kSkWBytes = 128 * 64 * 2, kSkXBytes = 64 * 64 * 2, kSkStage = kSkWBytes + kSkXBytes;
constexpr int kSkPitch = 132;          // floats between the batch rows of a parked partial tile (64 x 128 used)
constexpr int kSkNormBytes = 16384;     // the norm weight of up to 8192 k values, staged in shared memory
constexpr int kRowSqPitch = 320;       // floats between the batch rows of the sums-of-squares slots (>= 2 * 148 CTAs)
// The partial tile is parked over the pipeline's stages (dead once the last product has read them): a
// CTA takes under half of an SM's shared memory, so the next kernel of a chain starts -- and
// streams its first weight tiles -- beside this one.
constexpr int kSkSmem = kSkStages * kSkStage + 512 + 1024, kSkSmemDeep = kSkMaxStages * kSkStage + 512 + 1024;
static_assert(64 * kSkPitch * 4 <= kSkStages * kSkStage, "the parked tile must fit in the stages");

struct SkinnyParams {
  __nv_bfloat16* C;                   // (rows, N), ldc
  const __nv_bfloat16* residual;      // optional, C's shape and pitch
  int rows, N, K, ldc;
  int dual;                           // gated: tile = 64 gate rows + 64 up rows, N = output features
  int tiles, num_kb;
  int stages;                         // pipeline depth of this launch
  int* status;
  // RMSNorm folded in: every X tile is normalised in shared memory before the products read it
  const __nv_bfloat16* norm_w;
  const float* sq_in;                 // [64][kRowSqPitch]: sq_parts slots a row, left by the producing projection
  int sq_parts;
  float eps;
  float* sq_out;                      // this launch's slot per row: sum of squares of what it wrote (residual form)
  // RoPE + cache write folded in (q/k/v form): C is not written
  int rope_half;                      // 0, or D / 2
  const __nv_bfloat16* angles;
  const int* positions;
  __nv_bfloat16 *q_out, *k_cache, *v_cache;
  long long kv_batch_stride;
  int H, G, D, S;
};

// Two packed bf16 values x, scaled by `inv` in float32 and rounded, times two packed bf16 weights.
__device__ __forceinline__ uint32_t norm_pair(uint32_t x, uint32_t w, float inv) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(bf16_lo(x) * inv, bf16_hi(x) * inv);
  const __nv_bfloat162 y = __hmul2(h, *reinterpret_cast<const __nv_bfloat162*>(&w));
  return *reinterpret_cast<const uint32_t*>(&y);
}

// kFolds = false is the plain product: the folded forms' branches are compiled out of it (they cost it
// 4 to 15 % when they were not).
template <bool kFolds>
__global__ void __launch_bounds__(kSkThreads, 1)
gemm_skinny_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_w2,
                   const __grid_constant__ CUtensorMap map_x, const SkinnyParams p) {
  extern __shared__ uint8_t sk_raw[];
  const float* const sq_in = kFolds ? p.sq_in : nullptr;
  float* const sq_out = kFolds ? p.sq_out : nullptr;
  const int rope_half = kFolds ? p.rope_half : 0;
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(sk_raw) + 1023) & ~uintptr_t(1023));
  float* part = reinterpret_cast<float*>(smem);     // [batch row][feature], over the stages
  const int stages = p.stages;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + stages * kSkStage);
  uint64_t* full = bars;                     // [stages]
  uint64_t* empty = bars + kSkMaxStages;     // [stages]
  uint64_t* acc_full = empty + kSkMaxStages; // [1]
  // folded RMSNorm: X lands on a barrier of its own (from L2, long before the stage's weights from HBM),
  // is normalised in place, and the products wait for both
  uint64_t* x_full = acc_full + 1;           // [stages]
  uint64_t* ready = x_full + kSkMaxStages;   // [stages]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(ready + kSkMaxStages);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  uint8_t* norm_sm = smem + stages * kSkStage + 512;   // this rank's k range of the norm weight (folded RMSNorm)

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  cg::cluster_group cluster = cg::this_cluster();
  const int S = (int)cluster.num_blocks(), rank = (int)cluster.block_rank();
  const int tile = blockIdx.x / S;
  // this CTA's share of the k blocks
  const int per = (p.num_kb + S - 1) / S;
  const int kb_lo = min(p.num_kb, rank * per), kb_hi = min(p.num_kb, kb_lo + per);
  const int nkb = kb_hi - kb_lo;
  auto kblock = [&](int i) { return kb_lo + i; };    // the i-th k block this CTA takes
  const int rows_w = p.dual ? 64 : 128;          // output features a tile covers
  const int n0 = tile * rows_w;

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(full + s, 1); mbar_init(empty + s, 1);
      if (kFolds) { mbar_init(x_full + s, 1); mbar_init(ready + s, 4); }
    }
    mbar_init(acc_full, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w2) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(64)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_launch();

  auto load_w = [&](int stage, int kb) {
    uint8_t* dst = smem + stage * kSkStage;
    if (p.dual) {
      tma_load_2d(dst, &map_w, kb * 64, n0, full + stage);
      tma_load_2d(dst + 64 * 128, &map_w2, kb * 64, n0, full + stage);
    } else {
      tma_load_2d(dst, &map_w, kb * 64, n0, full + stage);
    }
  };

  int pos_first0 = 0, pos_first1 = 0;
  if (warp == 0) {
    // ---------------- producer ----------------
    if (lane == 0) {
      // the weights do not depend on the kernel before: the first stages' tiles go out ahead of the wait
      const bool own_x = sq_in != nullptr;       // X on its own barrier
      const uint32_t w_bytes = own_x ? kSkWBytes : kSkStage;
      int pre = 0;
      for (; pre < nkb && pre < stages; ++pre) {
        mbar_expect_tx(full + pre, w_bytes);
        load_w(pre, kblock(pre));
      }
      pdl_wait();
      int s = 0;
      uint32_t phase = 0;
      int issued = 0;
      for (; issued < nkb; ++issued) {
        const int kb = kblock(issued);
        if (issued >= pre) {
          if (!mbar_wait(empty + s, phase ^ 1, abort_flag)) break;
          mbar_expect_tx(full + s, w_bytes);
          load_w(s, kb);
        }
        if (own_x) mbar_expect_tx(x_full + s, kSkXBytes);
        tma_load_2d(smem + s * kSkStage + kSkWBytes, &map_x, kb * 64, 0, own_x ? x_full + s : full + s);
        if (++s == stages) { s = 0; phase ^= 1; }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      // bf16 x bf16 -> f32, M 128 (weight rows), N 64 (the batch), both operands K-major
      constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(64 >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
      int s = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int i = 0; i < nkb; ++i) {
        if (!mbar_wait(full + s, phase, abort_flag) || (sq_in && !mbar_wait(ready + s, phase, abort_flag))) { ok = false; break; }
        tcgen05_fence_after();
        const uint32_t w_addr = smem_u32(smem + s * kSkStage);
#pragma unroll
        for (int k = 0; k < 4; ++k)
          tcgen05_mma_bf16(tmem_base, make_desc(w_addr + k * 32, 16, 1024), make_desc(w_addr + kSkWBytes + k * 32, 16, 1024),
                           idesc, i != 0 || k != 0);
        tcgen05_commit(empty + s);
        if (++s == stages) { s = 0; phase ^= 1; }
      }
      if (ok) tcgen05_commit(acc_full);
    }
  } else {
    // ---------------- output warps: park this CTA's partial tile, row = tensor-memory lane ----------------
    if (sq_in) {   // the norm weight is a constant: staged ahead of the dependency wait
      const uint4* src = reinterpret_cast<const uint4*>(p.norm_w + (size_t)kb_lo * 64);
      for (int i = threadIdx.x - 64; i < (kb_hi - kb_lo) * 8; i += 128) reinterpret_cast<uint4*>(norm_sm)[i] = ld_cached(src + i);
      asm volatile("bar.sync 1, 128;" ::: "memory");
    }
    pdl_wait();
    if (rope_half) {    // the positions of this thread's first two items, fetched while the products run
      const int fq = (64 / S) >> 2, total = fq * p.rows, t = threadIdx.x - 64;
      if (t < total) pos_first0 = p.positions[t / fq];
      if (t + 128 < total) pos_first1 = p.positions[(t + 128) / fq];
    }
    if (sq_in) {
      // ---- the B operand, normalised in place: thread (row b, half kh) owns 32 of a k block's 64 values ----
      const int t = threadIdx.x - 64, b = t >> 1, kh = t & 1;
      float sum = 0.f;
      if (b < p.rows) {
        // sixteen 16-byte loads in flight at a time (a load is ~700 clocks away): 128 slots take one round
        const float* slots = sq_in + (size_t)b * kRowSqPitch;
        for (int base = kh * 4; base < p.sq_parts; base += 128) {
          float4 v[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int i = base + 8 * j;
            v[j] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (i + 4 <= p.sq_parts) v[j] = *reinterpret_cast<const float4*>(slots + i);
            else if (i < p.sq_parts) {
              v[j].x = slots[i];
              if (i + 1 < p.sq_parts) v[j].y = slots[i + 1];
              if (i + 2 < p.sq_parts) v[j].z = slots[i + 2];
            }
          }
#pragma unroll
          for (int j = 0; j < 16; ++j) { sum += v[j].x; sum += v[j].y; sum += v[j].z; sum += v[j].w; }
        }
      }
      const float s0 = __shfl_sync(0xffffffffu, sum, lane & ~1), s1 = __shfl_sync(0xffffffffu, sum, lane | 1);
      const float inv = 1.0f / sqrtf((s0 + s1) / (float)p.K + p.eps);
      int s = 0;
      uint32_t phase = 0;
      for (int i = 0; i < nkb; ++i) {
        const int kb = kblock(i);
        uint4 gw[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) gw[j] = *reinterpret_cast<const uint4*>(norm_sm + (kb - kb_lo) * 128 + kh * 64 + j * 16);
        if (!mbar_wait(x_full + s, phase, abort_flag)) break;
        uint8_t* xt = smem + s * kSkStage + kSkWBytes + b * 128;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint4* at = reinterpret_cast<uint4*>(xt + (((kh * 4 + j) ^ (b & 7)) << 4));   // the 128-byte swizzle
          const uint4 x = *at;
          // bf16(x / rms) by the conversion, times the weight as a bf16 product (one rounding, like the
          // float product of two bf16 values rounded): the norm kernel's two roundings
          uint4 o;
          o.x = norm_pair(x.x, gw[j].x, inv); o.y = norm_pair(x.y, gw[j].y, inv);
          o.z = norm_pair(x.z, gw[j].z, inv); o.w = norm_pair(x.w, gw[j].w, inv);
          *at = o;
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(ready + s);
        if (++s == stages) { s = 0; phase ^= 1; }
      }
    }
    const int q = warp & 3, n = q * 32 + lane;
    const bool have = kb_lo < kb_hi && mbar_wait(acc_full, 0, abort_flag);   // the products are done: the stages are free
    tcgen05_fence_after();
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      uint32_t v[32];
      if (have) {
        tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + 32 * half, v);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = 0u;       // no k blocks for this rank, or a wait gave up
      }
#pragma unroll
      for (int j = 0; j < 32; ++j) part[(size_t)(32 * half + j) * kSkPitch + n] = __uint_as_float(v[j]);
    }
  }
  tcgen05_fence_before();
  cluster.sync();      // every rank's partial tile is parked

  if (warp >= 2) {
    // ---- this rank's share of the tile, four features (or four rotation pairs) a thread, summed over
    // the ranks in order: all of a group's loads are issued before any is used (a remote one takes ~500
    // clocks).  A thread's second run of four is the up half of a gated tile or the rotation partners. ----
    const int t = threadIdx.x - 64;                 // 0 .. 127
    const bool two = p.dual || rope_half;
    const int second = p.dual ? 64 : rope_half;   // distance of the second run
    const int firsts = two ? 64 : 128;              // first runs' features in a tile
    const int feats = firsts / S, fq = feats >> 2, total = fq * p.rows;
    const float* src[8];
#pragma unroll
    for (int r = 0; r < 8; ++r) src[r] = (r < S && S > 1) ? cluster.map_shared_rank(part, r) : part;
    for (int g0 = 0; g0 < total; g0 += 128) {       // warp-uniform trips: the row sums below shuffle
      const int g = g0 + t;
      const int b = g / fq, first = rank * feats + 4 * (g - b * fq);
      // a rotation pair's low element: head (first / half) of the tile, element (first % half)
      const int f = rope_half ? (first / rope_half) * p.D + first % rope_half : first;
      const int col = n0 + f;
      const bool act = g < total && col < p.N;
      float sq = 0.f;
      if (act) {
        float4 va[8], vb[8];
        int pos = 0;
        uint4 turn = make_uint4(0u, 0u, 0u, 0u);
        if (rope_half) {     // the angle chunk is asked for before the partial tiles
          const int it = g0 >> 7;
          pos = it == 0 ? pos_first0 : it == 1 ? pos_first1 : p.positions[b];
          pos = max(0, min(pos, p.S - 1));
          if (col / p.D < p.H + p.G) turn = ld_cached(p.angles + (size_t)pos * p.D + 2 * (col % p.D));
        }
#pragma unroll
        for (int r = 0; r < 8; ++r)
          if (r < S) {
            va[r] = *reinterpret_cast<const float4*>(src[r] + (size_t)b * kSkPitch + f);
            if (two) vb[r] = *reinterpret_cast<const float4*>(src[r] + (size_t)b * kSkPitch + f + second);
          }
        float acc[4] = {0.f, 0.f, 0.f, 0.f}, acc2[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int r = 0; r < 8; ++r)
          if (r < S) {
            acc[0] += va[r].x; acc[1] += va[r].y; acc[2] += va[r].z; acc[3] += va[r].w;
            if (two) { acc2[0] += vb[r].x; acc2[1] += vb[r].y; acc2[2] += vb[r].z; acc2[3] += vb[r].w; }
          }
        float v[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) v[e] = round_bf16(acc[e]);
        if (rope_half) {
          // q and k heads turn by the angle row of this sequence's position; q goes out densely, k and v
          // into row `position` of the sequence's caches (the values the separate kernels would read and write)
          float w[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) w[e] = round_bf16(acc2[e]);
          const int hh = col / p.D, i0 = col - hh * p.D;
          if (hh < p.H + p.G) {
            float cs[8];
            unpack8(turn, cs);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float c = cs[2 * e], sn = cs[2 * e + 1];
              const float ya = __fsub_rn(__fmul_rn(v[e], c), __fmul_rn(w[e], sn));
              const float yb = __fadd_rn(__fmul_rn(w[e], c), __fmul_rn(v[e], sn));
              v[e] = ya; w[e] = yb;
            }
          }
          __nv_bfloat16* dst;
          if (hh < p.H) dst = p.q_out + ((size_t)b * p.H + hh) * p.D;
          else if (hh < p.H + p.G) dst = p.k_cache + (size_t)b * p.kv_batch_stride + ((size_t)pos * p.G + (hh - p.H)) * p.D;
          else dst = p.v_cache + (size_t)b * p.kv_batch_stride + ((size_t)pos * p.G + (hh - p.H - p.G)) * p.D;
          *reinterpret_cast<uint2*>(dst + i0) = make_uint2(pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3]));
          *reinterpret_cast<uint2*>(dst + i0 + rope_half) = make_uint2(pack_bf16x2(w[0], w[1]), pack_bf16x2(w[2], w[3]));
        } else {
          if (p.dual) {
#pragma unroll
            for (int e = 0; e < 4; ++e) v[e] = __fmul_rn(round_bf16(silu_f32(v[e])), round_bf16(acc2[e]));
          }
          const size_t off = (size_t)b * p.ldc + col;
          if (col + 4 <= p.N && (p.ldc & 3) == 0) {
            if (p.residual) {
              const uint2 rr = *reinterpret_cast<const uint2*>(p.residual + off);
              v[0] = __fadd_rn(v[0], bf16_lo(rr.x)); v[1] = __fadd_rn(v[1], bf16_hi(rr.x));
              v[2] = __fadd_rn(v[2], bf16_lo(rr.y)); v[3] = __fadd_rn(v[3], bf16_hi(rr.y));
            }
            if (sq_out) {
#pragma unroll
              for (int e = 0; e < 4; ++e) { v[e] = round_bf16(v[e]); sq = fmaf(v[e], v[e], sq); }
            }
            *reinterpret_cast<uint2*>(p.C + off) = make_uint2(pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3]));
          } else {
            for (int e = 0; e < 4 && col + e < p.N; ++e) {
              float w = v[e];
              if (p.residual) w = __fadd_rn(w, __bfloat162float(p.residual[off + e]));
              w = round_bf16(w);
              sq = fmaf(w, w, sq);
              p.C[off + e] = __float2bfloat16_rn(w);
            }
          }
        }
      }
      if (sq_out) {
        // the fq threads of a batch row are neighbours in a warp: one slot per (row, CTA), in a fixed order
        for (int m = 1; m < fq; m <<= 1) sq += __shfl_xor_sync(0xffffffffu, sq, m);
        if (g < total && g == b * fq) sq_out[(size_t)b * kRowSqPitch + blockIdx.x] = sq;
      }
    }
  }
  cluster.sync();      // nobody leaves while a peer still reads its tile
  if (threadIdx.x == 0 && *abort_flag && p.status) *p.status = IRON_ERR_TIMEOUT;
  if (warp == 1) {
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(64) : "memory");
  }
}

typedef CUresult (*SkEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                               const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                               CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static SkEncodeFn sk_encode() {
  static SkEncodeFn fn = nullptr;
  if (!fn) {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<SkEncodeFn>(sym);
  }
  return fn;
}
static bool sk_map(CUtensorMap* map, const void* base, uint64_t inner, uint64_t outer, uint64_t pitch, uint32_t box_outer) {
  SkEncodeFn fn = sk_encode();
  if (!fn) return false;
  const cuuint64_t dims[2] = {inner, outer};
  const cuuint64_t strides[1] = {pitch * 2};
  const cuuint32_t box[2] = {64, box_outer};
  const cuuint32_t elem[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// What a launch folds in beside the product (all optional).
struct SkinnyFold {
  const void* norm_w = nullptr;       // RMSNorm of X first: its weight, the producing projection's slots, eps
  const float* sq_in = nullptr;
  int sq_parts = 0;
  float eps = 0.f;
  float* sq_out = nullptr;            // leave this launch's sums of squares (residual form)
  // RoPE + cache write of a q/k/v projection
  const void* angles = nullptr;
  const int* positions = nullptr;
  void *q_out = nullptr, *k_cache = nullptr, *v_cache = nullptr;
  long long kv_batch_stride = 0;
  int H = 0, G = 0, D = 0, S = 0;
};

// How a product of this shape is laid over the machine: tiles and the K split.
static bool sk_plan(int rows, int N, int K, bool dual, int* tiles_out, int* split_out) {
  if (rows < 1 || rows > 64 || N < 1 || K < 64) return false;
  const int rows_w = dual ? 64 : 128;
  const int tiles = (N + rows_w - 1) / rows_w;
  if (tiles > 2 * kSMs) return false;   // many tiles (a head): the persistent GEMM amortises its prologue
  const int num_kb = (K + 63) / 64;
  // split K over a cluster while the machine is not yet full and a rank keeps at least four k blocks
  int S = 1;
  while (S < 8 && tiles * S * 2 <= kSMs && num_kb / (S * 2) >= 4) S *= 2;
  *tiles_out = tiles;
  *split_out = S;
  return true;
}

// X (rows <= 64, K) with pitch ldx; W (and W2 for the gated form) (N, K) with pitch ldw; C (rows, N).
// IRON_ERR_UNSUPPORTED when the shape is not this kernel's (the caller takes the general GEMM).
static int launch_skinny(const void* X, const void* W, const void* W2, void* C, const void* residual, int rows, int N,
                         int K, int ldx, int ldw, int ldc, const SkinnyFold& fold, int* d_status, cudaStream_t stream) {
  static const bool enabled = [] {
    const char* e = getenv("IRON_GEMM_SKINNY");
    return !(e && e[0] == '0');
  }();
  const bool dual = W2 != nullptr;
  int tiles = 0, S = 1;
  if (!enabled || !sk_plan(rows, N, K, dual, &tiles, &S)) return IRON_ERR_UNSUPPORTED;
  const int rows_w = dual ? 64 : 128;
  const int num_kb = (K + 63) / 64;
  CUtensorMap mw, mw2, mx;
  if (!sk_map(&mw, W, (uint64_t)K, (uint64_t)N, (uint64_t)ldw, (uint32_t)rows_w) ||
      !sk_map(&mw2, dual ? W2 : W, (uint64_t)K, (uint64_t)N, (uint64_t)ldw, (uint32_t)rows_w) ||
      !sk_map(&mx, X, (uint64_t)K, (uint64_t)rows, (uint64_t)ldx, 64))
    return IRON_ERR_LAUNCH;
  SkinnyParams p = {};
  p.C = (__nv_bfloat16*)C; p.residual = (const __nv_bfloat16*)residual;
  p.rows = rows; p.N = N; p.K = K; p.ldc = ldc; p.dual = dual ? 1 : 0; p.tiles = tiles; p.num_kb = num_kb;
  p.stages = S == 1 ? kSkMaxStages : kSkStages;
  p.status = d_status;
  p.norm_w = (const __nv_bfloat16*)fold.norm_w; p.sq_in = fold.sq_in; p.sq_parts = fold.sq_parts; p.eps = fold.eps;
  p.sq_out = fold.sq_out;
  if (fold.angles) {
    p.rope_half = fold.D / 2;
    p.angles = (const __nv_bfloat16*)fold.angles; p.positions = fold.positions;
    p.q_out = (__nv_bfloat16*)fold.q_out; p.k_cache = (__nv_bfloat16*)fold.k_cache; p.v_cache = (__nv_bfloat16*)fold.v_cache;
    p.kv_batch_stride = fold.kv_batch_stride; p.H = fold.H; p.G = fold.G; p.D = fold.D; p.S = fold.S;
  }
  const bool folds = fold.norm_w || fold.sq_out || fold.angles;
  static DeviceOnce configured;   // the attribute is per device
  if (!configured.done()) {
    if (cudaFuncSetAttribute(gemm_skinny_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSkSmemDeep) != cudaSuccess ||
        cudaFuncSetAttribute(gemm_skinny_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSkSmemDeep + kSkNormBytes) != cudaSuccess)
      return IRON_ERR_LAUNCH;
    configured.mark();
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(tiles * S);
  cfg.blockDim = dim3(kSkThreads);
  // with the norm folded in, a rank's k range of the norm weight sits behind the stages
  const int per = (num_kb + S - 1) / S;
  cfg.dynamicSmemBytes = (S == 1 ? kSkSmemDeep : kSkSmem) + (fold.sq_in ? per * 128 : 0);
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = S;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1 + pdl_attr_count();
  const cudaError_t e = folds ? cudaLaunchKernelEx(&cfg, gemm_skinny_kernel<true>, mw, mw2, mx, p)
                              : cudaLaunchKernelEx(&cfg, gemm_skinny_kernel<false>, mw, mw2, mx, p);
  return e == cudaSuccess ? IRON_OK : IRON_ERR_LAUNCH;
}

int launch_gemm_skinny(const void* X, const void* W, const void* W2, void* C, const void* residual, int rows, int N,
                       int K, int ldx, int ldw, int ldc, int* d_status, cudaStream_t stream) {
  return launch_skinny(X, W, W2, C, residual, rows, N, K, ldx, ldw, ldc, SkinnyFold{}, d_status, stream);
}

}  // namespace iron

using namespace iron;

extern "C" int iron_gemm_rows_parts(int rows, int N, int K, int gated) {
  int tiles = 0, S = 1;
  if (!sk_plan(rows, N, K, gated != 0, &tiles, &S)) return 0;
  return tiles * S;
}

// the checks the folded norm shares between the two entry points
static int check_norm(const void* X, const void* norm_weight, const float* d_rowsq_in, int rowsq_parts, int K, int ldx) {
  if (!norm_weight && !d_rowsq_in) return IRON_OK;
  if (!norm_weight || !d_rowsq_in) return IRON_ERR_SHAPE;
  if (rowsq_parts < 1 || rowsq_parts > kRowSqPitch || (K & 63) || (ldx & 7)) return IRON_ERR_SHAPE;
  if (K * 2 > kSkNormBytes) return IRON_ERR_UNSUPPORTED;
  if (!aligned16(X) || !aligned16(norm_weight) || !aligned16(d_rowsq_in)) return IRON_ERR_ALIGN;
  return IRON_OK;
}

extern "C" int iron_gemm_rows_bf16(const void* X, const void* W, const void* W2, void* C, const void* residual,
                                   int rows, int N, int K, int ldx, int ldw, int ldc, const void* norm_weight,
                                   const float* d_rowsq_in, int rowsq_parts, float eps, float* d_rowsq_out,
                                   int* d_status, iron_stream_t stream) {
  if (rows < 0 || rows > 64 || N <= 0 || K <= 0 || (K & 7)) return IRON_ERR_SHAPE;
  if (!X || !W || !C) return IRON_ERR_SHAPE;
  if (ldx < K || ldw < K || ldc < N || (ldx & 7) || (ldw & 7)) return IRON_ERR_SHAPE;
  if (!aligned16(X) || !aligned16(W) || (W2 && !aligned16(W2)) || !aligned16(C) || (residual && !aligned16(residual)))
    return IRON_ERR_ALIGN;
  if (W2 && residual) return IRON_ERR_SHAPE;                        // the gated form has no residual
  if (d_rowsq_out && (W2 || !residual || !aligned16(d_rowsq_out))) return IRON_ERR_SHAPE;   // sums of the residual stream only
  const int rc = check_norm(X, norm_weight, d_rowsq_in, rowsq_parts, K, ldx);
  if (rc != IRON_OK) return rc;
  if (rows == 0) return IRON_OK;
  SkinnyFold fold;
  fold.norm_w = norm_weight; fold.sq_in = d_rowsq_in; fold.sq_parts = rowsq_parts; fold.eps = eps;
  fold.sq_out = d_rowsq_out;
  return launch_skinny(X, W, W2, C, residual, rows, N, K, ldx, ldw, ldc, fold, d_status, (cudaStream_t)stream);
}

extern "C" int iron_gemm_rows_qkv_rope_bf16(const void* X, const void* Wqkv, int rows, int K, int ldx, int ldw,
                                            const void* norm_weight, const float* d_rowsq_in, int rowsq_parts,
                                            float eps, const void* angles, const int* d_positions, void* q_out,
                                            void* k_cache, void* v_cache, long long kv_batch_stride, int H, int G,
                                            int D, int S, int* d_status, iron_stream_t stream) {
  if (rows < 0 || rows > 64 || K <= 0 || (K & 7) || H <= 0 || G <= 0 || S <= 0) return IRON_ERR_SHAPE;
  if (D != 64 && D != 128) return IRON_ERR_UNSUPPORTED;              // a 128-row tile holds whole heads
  const long long N = (long long)(H + 2 * G) * D;
  if ((N & 127) || ((long long)H * D & 127) || ((long long)G * D & 127)) return IRON_ERR_UNSUPPORTED;
  if (!X || !Wqkv || !angles || !d_positions || !q_out || !k_cache || !v_cache) return IRON_ERR_SHAPE;
  if (ldx < K || ldw < K || (ldx & 7) || (ldw & 7) || (kv_batch_stride & 7)) return IRON_ERR_SHAPE;
  if (!aligned16(X) || !aligned16(Wqkv) || !aligned16(angles) || !aligned16(q_out) || !aligned16(k_cache) ||
      !aligned16(v_cache))
    return IRON_ERR_ALIGN;
  const int rc = check_norm(X, norm_weight, d_rowsq_in, rowsq_parts, K, ldx);
  if (rc != IRON_OK) return rc;
  if (rows == 0) return IRON_OK;
  SkinnyFold fold;
  fold.norm_w = norm_weight; fold.sq_in = d_rowsq_in; fold.sq_parts = rowsq_parts; fold.eps = eps;
  fold.angles = angles; fold.positions = d_positions; fold.q_out = q_out; fold.k_cache = k_cache; fold.v_cache = v_cache;
  fold.kv_batch_stride = kv_batch_stride; fold.H = H; fold.G = G; fold.D = D; fold.S = S;
  return launch_skinny(X, Wqkv, nullptr, q_out, nullptr, rows, (int)N, K, ldx, ldw, (int)N, fold, d_status,
                       (cudaStream_t)stream);
}
