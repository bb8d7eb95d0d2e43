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
// The partial tile is parked over the pipeline's stages (dead once the last product has read them): a
// CTA takes under half of an SM's shared memory, so the next kernel of a chain starts -- and
// streams its first weight tiles -- beside this one.
constexpr int kSkSmem = kSkStages * kSkStage + 256 + 1024, kSkSmemDeep = kSkMaxStages * kSkStage + 256 + 1024;
static_assert(64 * kSkPitch * 4 <= kSkStages * kSkStage, "the parked tile must fit in the stages");

struct SkinnyParams {
  __nv_bfloat16* C;                   // (rows, N), ldc
  const __nv_bfloat16* residual;      // optional, C's shape and pitch
  int rows, N, K, ldc;
  int dual;                           // gated: tile = 64 gate rows + 64 up rows, N = output features
  int tiles, num_kb;
  int stages;                         // pipeline depth of this launch
  int* status;
};

__global__ void __launch_bounds__(kSkThreads, 1)
gemm_skinny_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_w2,
                   const __grid_constant__ CUtensorMap map_x, const SkinnyParams p) {
  extern __shared__ uint8_t sk_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(sk_raw) + 1023) & ~uintptr_t(1023));
  float* part = reinterpret_cast<float*>(smem);     // [batch row][feature], over the stages
  const int stages = p.stages;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + stages * kSkStage);
  uint64_t* full = bars;                     // [stages]
  uint64_t* empty = bars + kSkMaxStages;     // [stages]
  uint64_t* acc_full = empty + kSkMaxStages; // [1]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  cg::cluster_group cluster = cg::this_cluster();
  const int S = (int)cluster.num_blocks(), rank = (int)cluster.block_rank();
  const int tile = blockIdx.x / S;
  // this CTA's share of the k blocks
  const int per = (p.num_kb + S - 1) / S;
  const int kb_lo = min(p.num_kb, rank * per), kb_hi = min(p.num_kb, kb_lo + per);
  const int rows_w = p.dual ? 64 : 128;          // output features a tile covers
  const int n0 = tile * rows_w;

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) { mbar_init(full + s, 1); mbar_init(empty + s, 1); }
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

  if (warp == 0) {
    // ---------------- producer ----------------
    if (lane == 0) {
      // the weights do not depend on the kernel before: the first stages' tiles go out ahead of the wait
      int pre = 0;
      for (int kb = kb_lo; kb < kb_hi && pre < stages; ++kb, ++pre) {
        mbar_expect_tx(full + pre, kSkStage);
        load_w(pre, kb);
      }
      pdl_wait();
      int s = 0;
      uint32_t phase = 0;
      int issued = 0;
      for (int kb = kb_lo; kb < kb_hi; ++kb, ++issued) {
        if (issued >= pre) {
          if (!mbar_wait(empty + s, phase ^ 1, abort_flag)) break;
          mbar_expect_tx(full + s, kSkStage);
          load_w(s, kb);
        }
        tma_load_2d(smem + s * kSkStage + kSkWBytes, &map_x, kb * 64, 0, full + s);
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
      for (int kb = kb_lo; kb < kb_hi; ++kb) {
        if (!mbar_wait(full + s, phase, abort_flag)) { ok = false; break; }
        tcgen05_fence_after();
        const uint32_t w_addr = smem_u32(smem + s * kSkStage);
#pragma unroll
        for (int k = 0; k < 4; ++k)
          tcgen05_mma_bf16(tmem_base, make_desc(w_addr + k * 32, 16, 1024), make_desc(w_addr + kSkWBytes + k * 32, 16, 1024),
                           idesc, kb != kb_lo || k != 0);
        tcgen05_commit(empty + s);
        if (++s == stages) { s = 0; phase ^= 1; }
      }
      if (ok) tcgen05_commit(acc_full);
    }
  } else {
    // ---------------- output warps: park this CTA's partial tile, row = tensor-memory lane ----------------
    pdl_wait();
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
    // ---- this rank's share of the tile's output features, four at a time, summed over the ranks in
    // order: all of a group's loads are issued before any is used (a remote one takes ~500 clocks) ----
    const int t = threadIdx.x - 64;                 // 0 .. 127
    const int feats = rows_w / S, f0 = rank * feats, fq = feats >> 2;
    const float* src[8];
#pragma unroll
    for (int r = 0; r < 8; ++r) src[r] = (r < S && S > 1) ? cluster.map_shared_rank(part, r) : part;
    for (int g = t; g < fq * p.rows; g += 128) {
      const int b = g / fq, f = f0 + 4 * (g - b * fq);
      const int col = n0 + f;
      if (col >= p.N) continue;
      float4 va[8], vb[8];
#pragma unroll
      for (int r = 0; r < 8; ++r)
        if (r < S) {
          va[r] = *reinterpret_cast<const float4*>(src[r] + (size_t)b * kSkPitch + f);
          if (p.dual) vb[r] = *reinterpret_cast<const float4*>(src[r] + (size_t)b * kSkPitch + f + 64);
        }
      float acc[4] = {0.f, 0.f, 0.f, 0.f}, acc2[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int r = 0; r < 8; ++r)
        if (r < S) {
          acc[0] += va[r].x; acc[1] += va[r].y; acc[2] += va[r].z; acc[3] += va[r].w;
          if (p.dual) { acc2[0] += vb[r].x; acc2[1] += vb[r].y; acc2[2] += vb[r].z; acc2[3] += vb[r].w; }
        }
      const size_t off = (size_t)b * p.ldc + col;
      float v[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        v[e] = round_bf16(acc[e]);
        if (p.dual) v[e] = __fmul_rn(round_bf16(silu_f32(v[e])), round_bf16(acc2[e]));
      }
      if (col + 4 <= p.N && (p.ldc & 3) == 0) {
        if (p.residual) {
          const uint2 rr = *reinterpret_cast<const uint2*>(p.residual + off);
          v[0] = __fadd_rn(v[0], bf16_lo(rr.x)); v[1] = __fadd_rn(v[1], bf16_hi(rr.x));
          v[2] = __fadd_rn(v[2], bf16_lo(rr.y)); v[3] = __fadd_rn(v[3], bf16_hi(rr.y));
        }
        *reinterpret_cast<uint2*>(p.C + off) = make_uint2(pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3]));
      } else {
        for (int e = 0; e < 4 && col + e < p.N; ++e) {
          float w = v[e];
          if (p.residual) w = __fadd_rn(w, __bfloat162float(p.residual[off + e]));
          p.C[off + e] = __float2bfloat16_rn(w);
        }
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

// X (rows <= 64, K) with pitch ldx; W (and W2 for the gated form) (N, K) with pitch ldw; C (rows, N).
// IRON_ERR_UNSUPPORTED when the shape is not this kernel's (the caller takes the general GEMM).
int launch_gemm_skinny(const void* X, const void* W, const void* W2, void* C, const void* residual, int rows, int N,
                       int K, int ldx, int ldw, int ldc, int* d_status, cudaStream_t stream) {
  static const bool enabled = [] {
    const char* e = getenv("IRON_GEMM_SKINNY");
    return !(e && e[0] == '0');
  }();
  if (!enabled || rows < 1 || rows > 64 || N < 1 || K < 64) return IRON_ERR_UNSUPPORTED;
  const bool dual = W2 != nullptr;
  const int rows_w = dual ? 64 : 128;
  const int tiles = (N + rows_w - 1) / rows_w;
  if (tiles > 2 * kSMs) return IRON_ERR_UNSUPPORTED;   // many tiles (a head): the persistent GEMM amortises its prologue
  const int num_kb = (K + 63) / 64;
  // split K over a cluster while the machine is not yet full and a rank keeps at least four k blocks
  int S = 1;
  while (S < 8 && tiles * S * 2 <= kSMs && num_kb / (S * 2) >= 4) S *= 2;
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
  static DeviceOnce configured;   // the attribute is per device
  if (!configured.done()) {
    if (cudaFuncSetAttribute(gemm_skinny_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSkSmemDeep) != cudaSuccess)
      return IRON_ERR_LAUNCH;
    configured.mark();
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(tiles * S);
  cfg.blockDim = dim3(kSkThreads);
  cfg.dynamicSmemBytes = S == 1 ? kSkSmemDeep : kSkSmem;
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
  return cudaLaunchKernelEx(&cfg, gemm_skinny_kernel, mw, mw2, mx, p) == cudaSuccess ? IRON_OK : IRON_ERR_LAUNCH;
}

}  // namespace iron
