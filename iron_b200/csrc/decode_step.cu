// One decode step of a Llama-architecture model as ONE persistent kernel.
//
// At batch 1 a decode step is a chain of ~80 small dependent operations (per layer: QKV
// projection + RoPE + cache write, attention, o_proj, gate/up + SwiGLU, down_proj) whose
// only real cost is streaming 2.5 GB of weights.  Launched one by one, every link of the
// chain stops the weight stream for a few microseconds.  Here the whole step -- every
// layer, the final norm, the head and the greedy draw -- runs as phases of one cooperative
// grid, one CTA per SM, and the weight stream is decoupled from the chain:
//
//   * Every warp owns a private ring of shared-memory slots that the TMA engine fills with
//     bulk copies (cp.async.bulk + mbarrier complete_tx).  A warp's work items -- 256
//     columns of 8 consecutive weight rows -- form ONE static sequence over all phases of
//     the step, so the copies for the next phase are issued, and land, while the CTA is
//     still waiting for the previous phase to finish everywhere.
//   * An item (8 rows x 256 columns, 4 KB) arrives by ONE tiled TMA copy
//     (cp.async.bulk.tensor.2d through a tensor map of the weight matrix; two copies of
//     4 rows for the gate/up pair).  A lane multiplies its 8 columns of the staged
//     activation vector into all 8 rows with packed two-wide f32 FMAs, so the vector is
//     unpacked once per item and an item costs ~120 instructions per lane.
//   * The narrow projections (q/k/v, o_proj, down_proj) have too few 8-row groups to
//     occupy the grid, so their reduction dimension is split too: a unit is (row group,
//     K part), its result an f32 partial in global memory, and the *consumer* of the
//     projection sums the parts in a fixed order, rounds to bf16 and applies what follows
//     (residual add and RMSNorm in the next projection's staging; RoPE and the cache write
//     in the attention phase).  Results do not depend on the grid size or on timing.
//   * Phases are separated by a grid-wide barrier: a monotonically increasing counter in
//     global memory (zeroed by a memset node ahead of the kernel).  The launch is
//     cooperative, so every CTA is resident and the barrier cannot starve; every spin (on
//     the counter or on an mbarrier) is still bounded by a wall-clock limit, after which the
//     CTA records IRON_ERR_TIMEOUT in the status word, waits for its own copies in flight and
//     leaves, and every other CTA follows.
//
// Roundings are those of the separate kernels: f32 dot products rounded once to bf16,
// RMSNorm with its two roundings, RoPE on the rounded projections, the residual added
// after the rounding, SiLU and the product rounded separately.
#include <cuda.h>

#include "common.cuh"

namespace iron {

constexpr int kStepWarps = 16;
constexpr int kStepThreads = kStepWarps * 32;
constexpr int kItemRows = 8;                        // weight rows of one item
constexpr int kItemCols = 256;                      // columns of one item: 8 per lane
constexpr int kRowPitch = kItemCols * 2;            // bytes between rows in a slot
constexpr int kSlotBytes = kItemRows * kRowPitch;   // 4 KB
constexpr int kSlots = 3;                           // slots in a warp's ring (192 KB per CTA)
constexpr int kStepMaxK = 8192;                     // longest reduction (activation staging)
constexpr int kStepMaxParts = 8;                    // K parts of a narrow projection
constexpr int kStepMaxLayers = 64;                  // rows of the layer table in shared memory
constexpr int kMapsPerLayer = 5;                    // tensor maps: wqkv, wo, wg, wu, wd
constexpr unsigned long long kStepWaitNs = 2000000000ull;  // 2 s
constexpr size_t kStepRingBytes = (size_t)kStepWarps * kSlots * kSlotBytes;
constexpr size_t kStepBarsOff = kStepRingBytes + (size_t)kStepMaxK * 2;
constexpr size_t kStepTableOff = kStepBarsOff + kStepWarps * kSlots * 8;
constexpr size_t kStepSmem = kStepTableOff + (size_t)kStepMaxLayers * 9 * sizeof(void*);

struct StepLayer {
  const __nv_bfloat16 *ln1, *wqkv, *wo, *ln2, *wg, *wu, *wd;
  __nv_bfloat16 *k, *v;
};

struct StepParams {
  const StepLayer* layers;  // device array of L entries
  const CUtensorMap* maps;  // device array: 5 per layer (wqkv, wo, wg, wu, wd), then the head
  int L, E, F, H, G, D, V, S;
  const __nv_bfloat16 *embed, *head, *final_norm, *angles;
  float eps, scale_log2;
  int window;
  int* values;              // [token, position]; updated at the end
  int* drawn;               // (S)
  __nv_bfloat16 *xa, *xb, *act, *logits;
  float *part_qkv, *part_o, *part_d;   // (parts, rows) f32 partial sums
  int kp_qkv, kp_o, kp_d;   // K parts of the three narrow projections (powers of two)
  float* att_part;          // (H, nsplit, D + 4): D outputs, maximum, sum, padding
  int nsplit;
  unsigned int* barrier;
  unsigned long long* best; // one partial argmax key per CTA
  int* status;
  unsigned long long* trace; // CTA 0's timestamps: 3 per phase (waited, staged, items done)
};

// The layer table is copied to shared memory when the kernel starts: the item cursors look
// a layer's pointers up at every phase change, on the critical path.
__device__ __forceinline__ StepLayer* layer_table() {
  extern __shared__ __align__(128) unsigned char step_smem[];
  return reinterpret_cast<StepLayer*>(step_smem + kStepTableOff);
}

// ---- PTX wrappers ---------------------------------------------------------------------
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
__device__ __forceinline__ void step_stamp(const StepParams& sp, unsigned int epoch, int which) {
  if (blockIdx.x == 0 && threadIdx.x == 0 && epoch < 340u) sp.trace[3 * epoch + which] = step_ns();
}
__device__ __forceinline__ void step_mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void step_mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool step_mbar_try_wait(uint64_t* bar, uint32_t parity) {
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
__device__ __forceinline__ uint64_t step_evict_first_policy() {
  uint64_t pol;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}
// One box of a tensor map (rows x 256 columns from column x, row y) to this CTA's shared
// memory; completion is counted on `bar`.  The weights are read once per step: first in
// line for eviction from L2.  Columns and rows past the matrix arrive as zeros.
__device__ __forceinline__ void step_tensor_load(uint32_t dst, const CUtensorMap* map, int x, int y, uint64_t* bar,
                                                 uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint "
      "[%0], [%1, {%2, %3}], [%4], %5;"
      ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar)), "l"(policy)
      : "memory");
}
// (lo, hi) of a word holding two bf16, as f32
__device__ __forceinline__ float2 step_pair(uint32_t w) {
  return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
}

// ---- grid barrier, split into arrive and wait ----------------------------------------
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

struct StepShared {
  int abort;
  float red[32];
  unsigned long long best[kStepWarps];
  float att_ml[kStepWarps][2];
  alignas(16) float q[128];             // this CTA's query head: rotated, scaled (attention phase)
  alignas(16) __nv_bfloat16 knew[128];  // the new cache rows of this CTA's KV head
  alignas(16) __nv_bfloat16 vnew[128];
};

// ---- the static sequence of weight items ----------------------------------------------
// Phase ids: 4 per layer (QKV, o_proj, gate/up, down_proj), then the head.  The attention
// phase streams no weights and has no id.  A phase is cut into units that go round the
// grid's warps; a unit is cut into items of 8 rows x 256 columns.
//   PH_PART   a unit is (8-row group, K part); the result is an f32 partial per row.
//   PH_SWIGLU a unit is 4 rows of the gate matrix and the same 4 rows of the up matrix
//             (slot rows 0-3 and 4-7), over all of K; the result is bf16 silu(gate) * up.
//   PH_HEAD   a unit is an 8-row group over all of K; the result is a bf16 logit per row.
enum { PH_PART = 0, PH_SWIGLU = 1, PH_HEAD = 2 };

struct Phase {
  const CUtensorMap *map_a, *map_b;   // map_b: the up matrix of PH_SWIGLU
  float* part;                        // PH_PART: (parts, rows)
  int mode, units, K, rows, kshift, part_cols, nitems, first;
};

__device__ __forceinline__ Phase load_phase(const StepParams& sp, int pid, int gw, int NW) {
  Phase ph;
  const int rows_qkv = (sp.H + 2 * sp.G) * sp.D;
  const unsigned int u_qkv = (unsigned int)(rows_qkv >> 3) * (unsigned int)sp.kp_qkv;
  const unsigned int u_o = (unsigned int)(sp.E >> 3) * (unsigned int)sp.kp_o;
  const unsigned int u_sw = (unsigned int)(sp.F >> 2);
  const unsigned int u_d = (unsigned int)(sp.E >> 3) * (unsigned int)sp.kp_d;
  const int layer = pid >> 2, j = pid & 3;
  unsigned int before = (unsigned int)layer * (u_qkv + u_o + u_sw + u_d);   // units of every earlier phase
  int parts = 1;
  ph.map_b = nullptr; ph.part = nullptr;
  if (layer >= sp.L) {
    ph.map_a = sp.maps + kMapsPerLayer * sp.L; ph.mode = PH_HEAD; ph.rows = sp.V; ph.K = sp.E;
  } else {
    const CUtensorMap* m = sp.maps + kMapsPerLayer * layer;
    if (j == 0) { ph.map_a = m; ph.mode = PH_PART; ph.rows = rows_qkv; ph.K = sp.E; parts = sp.kp_qkv; ph.part = sp.part_qkv; }
    else if (j == 1) { ph.map_a = m + 1; ph.mode = PH_PART; ph.rows = sp.E; ph.K = sp.H * sp.D; parts = sp.kp_o; ph.part = sp.part_o; before += u_qkv; }
    else if (j == 2) { ph.map_a = m + 2; ph.map_b = m + 3; ph.mode = PH_SWIGLU; ph.rows = sp.F; ph.K = sp.E; before += u_qkv + u_o; }
    else { ph.map_a = m + 4; ph.mode = PH_PART; ph.rows = sp.E; ph.K = sp.F; parts = sp.kp_d; ph.part = sp.part_d; before += u_qkv + u_o + u_sw; }
  }
  ph.kshift = 31 - __clz(parts);
  ph.units = ph.mode == PH_SWIGLU ? (ph.rows >> 2) : ((ph.rows >> 3) << ph.kshift);
  ph.part_cols = (((ph.K >> ph.kshift) + 31) >> 5) << 5;
  ph.nitems = (ph.part_cols + kItemCols - 1) / kItemCols;
  // units go round the grid's warps, each phase starting where the one before stopped
  const int rot = (int)(before % (unsigned int)NW);
  ph.first = gw - rot + (gw < rot ? NW : 0);
  return ph;
}

// What an item covers: `group` counts 8-row groups (4-row groups of both matrices for
// PH_SWIGLU), the columns are [col0, col0 + ncols).
struct ItemGeom {
  int group, kpart, col0, ncols;
};
__device__ __forceinline__ ItemGeom item_geom(const Phase& ph, int unit, int item) {
  ItemGeom g;
  g.group = unit >> ph.kshift;
  g.kpart = unit - (g.group << ph.kshift);
  g.col0 = g.kpart * ph.part_cols + item * kItemCols;
  const int end = min(ph.K, (g.kpart + 1) * ph.part_cols);
  g.ncols = max(0, min(kItemCols, end - g.col0));
  return g;
}

// A position in a warp's item sequence.
struct Cursor {
  Phase ph;
  int pid, unit, item, idx;
  bool done;
};

__device__ __forceinline__ void cursor_seek(Cursor& c, const StepParams& sp, int gw, int NW) {
  // move to the next phase that has a unit for this warp
  const int NP = 4 * sp.L + 1;
  while (c.unit >= c.ph.units) {
    if (++c.pid >= NP) { c.done = true; return; }
    c.ph = load_phase(sp, c.pid, gw, NW);
    c.unit = c.ph.first;
  }
}
__device__ __forceinline__ void cursor_start(Cursor& c, const StepParams& sp, int gw, int NW) {
  c.pid = -1; c.unit = 0; c.item = 0; c.idx = 0; c.done = false;
  c.ph.units = 0;
  cursor_seek(c, sp, gw, NW);
}
__device__ __forceinline__ void cursor_advance(Cursor& c, const StepParams& sp, int gw, int NW) {
  ++c.idx;
  if (++c.item < c.ph.nitems) return;
  c.item = 0;
  c.unit += NW;
  cursor_seek(c, sp, gw, NW);
}

// What a warp carries through the step: its ring (slots filled by the TMA engine, one
// mbarrier per slot) and its two positions in the item sequence.
struct Stream {
  uint32_t slots;    // shared-memory address of kSlots x kSlotBytes
  uint64_t* bars;    // kSlots
  uint64_t policy;
  Cursor iss, con;   // the next item to start copying / to consume
  int gw, NW;        // this warp's index in the grid, warps in the grid
};

// Lane 0 starts the copy of the item at `st.iss` into the slot its index maps to.  A box
// always counts its full size on the mbarrier, zero fill included.
__device__ __forceinline__ void ring_issue(const Stream& st) {
  const Cursor& c = st.iss;
  const ItemGeom g = item_geom(c.ph, c.unit, c.item);
  const int s = c.idx % kSlots;
  const uint32_t dst = st.slots + s * kSlotBytes;
  step_mbar_expect_tx(st.bars + s, kSlotBytes);
  if (c.ph.mode == PH_SWIGLU) {
    step_tensor_load(dst, c.ph.map_a, g.col0, g.group * 4, st.bars + s, st.policy);
    step_tensor_load(dst + 4 * kRowPitch, c.ph.map_b, g.col0, g.group * 4, st.bars + s, st.policy);
  } else {
    step_tensor_load(dst, c.ph.map_a, g.col0, g.group * kItemRows, st.bars + s, st.policy);
  }
}

// Every lane waits for the item with index `idx` to have landed; false when out of time.
__device__ __forceinline__ bool ring_wait(const Stream& st, int idx, int* status, int* s_abort) {
  uint64_t* bar = st.bars + idx % kSlots;
  const uint32_t parity = (uint32_t)(idx / kSlots) & 1u;
  if (step_mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = step_ns();
  for (uint32_t it = 1;; ++it) {
    if (step_mbar_try_wait(bar, parity)) return true;
    if ((it & 63u) == 0 && step_ns() - t0 > kStepWaitNs) {
      *reinterpret_cast<volatile int*>(status) = IRON_ERR_TIMEOUT;
      *reinterpret_cast<volatile int*>(s_abort) = 1;
      return false;
    }
  }
}

enum { ST_VECTOR = 0, ST_PARTIAL = 1, ST_ATTENTION = 2 };

struct PhaseArgs {
  int mode;                          // PH_*
  int stage;                         // ST_*
  int K;                             // reduction length (the staged vector)
  const __nv_bfloat16* x;            // ST_VECTOR: the activation vector
  const float* parts;                // ST_PARTIAL: (nparts, K) partial sums of the projection before
  int nparts;
  const __nv_bfloat16* residual;     // ST_PARTIAL: added after the rounding
  __nv_bfloat16* keep;               // ST_PARTIAL: the sum is also the new residual stream (CTA 0 stores it)
  const __nv_bfloat16* norm_w;       // non-null: RMSNorm(x) * norm_w is staged
  __nv_bfloat16* y;                  // PH_SWIGLU, PH_HEAD: the output vector
};

// One weight phase: wait for the phase before, stage its result as this phase's activation
// vector, then every warp consumes the items of phase `pid` in its sequence -- re-arming
// each slot it frees with the next item of the sequence, whatever phase that belongs to.
// Whatever does not depend on the phase before (norm weights, the residual vector, which
// is at least two phases old) is fetched ahead of the wait.
__device__ __forceinline__ bool weight_phase(const StepParams& sp, int pid, const PhaseArgs& a, Stream& st,
                                             const unsigned char* ring_bytes, unsigned char* xs_bytes,
                                             StepShared& sh, unsigned int& epoch, unsigned long long& best) {
  constexpr int kIter = (kStepMaxK / 8 + kStepThreads - 1) / kStepThreads;
  const int tid = threadIdx.x, lane = tid & 31;
  const int K = a.K, nch = K >> 3;
  uint4* xs = reinterpret_cast<uint4*>(xs_bytes);

  uint4 wreg[kIter], rreg[kIter];
#pragma unroll
  for (int k = 0; k < kIter; ++k) {
    const int i = tid + k * kStepThreads;
    wreg[k] = make_uint4(0, 0, 0, 0);
    rreg[k] = make_uint4(0, 0, 0, 0);
    if (i < nch) {
      if (a.norm_w) wreg[k] = ld_cached(reinterpret_cast<const uint4*>(a.norm_w) + i);
      if (a.stage == ST_PARTIAL && a.residual) rreg[k] = __ldcg(reinterpret_cast<const uint4*>(a.residual) + i);
    }
  }

  if (!grid_wait(sp.barrier, epoch, sp.status, &sh.abort)) return false;
  step_stamp(sp, epoch, 0);

  // ---- stage the activation vector ----
  if (a.stage != ST_ATTENTION) {
    uint4 xreg[kIter];
    if (a.stage == ST_VECTOR) {
#pragma unroll
      for (int k = 0; k < kIter; ++k) {
        const int i = tid + k * kStepThreads;
        xreg[k] = i < nch ? __ldcg(reinterpret_cast<const uint4*>(a.x) + i) : make_uint4(0, 0, 0, 0);
      }
    } else {
      // the projection before left f32 partial sums: add them in a fixed order, round,
      // add the residual, round -- this is the new residual stream
#pragma unroll
      for (int k = 0; k < kIter; ++k) {
        const int i = tid + k * kStepThreads;
        xreg[k] = make_uint4(0, 0, 0, 0);
        if (i < nch) {
          float s[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll 4
          for (int p = 0; p < a.nparts; ++p) {
            const float4 lo = __ldcg(reinterpret_cast<const float4*>(a.parts + (size_t)p * K + i * 8));
            const float4 hi = __ldcg(reinterpret_cast<const float4*>(a.parts + (size_t)p * K + i * 8 + 4));
            s[0] += lo.x; s[1] += lo.y; s[2] += lo.z; s[3] += lo.w;
            s[4] += hi.x; s[5] += hi.y; s[6] += hi.z; s[7] += hi.w;
          }
          if (a.residual) {
            float r[8];
            unpack8(rreg[k], r);
#pragma unroll
            for (int j = 0; j < 8; ++j) s[j] = __fadd_rn(round_bf16(s[j]), r[j]);
          }
          xreg[k] = pack8(s);
          if (a.keep && blockIdx.x == 0) reinterpret_cast<uint4*>(a.keep)[i] = xreg[k];
        }
      }
    }
    if (a.norm_w) {
      float ss = 0.f;
#pragma unroll
      for (int k = 0; k < kIter; ++k) {
        float f[8];
        unpack8(xreg[k], f);
#pragma unroll
        for (int j = 0; j < 8; ++j) ss = fmaf(f[j], f[j], ss);
      }
      const float tot = block_sum(ss, sh.red);
      const float inv = 1.0f / sqrtf(tot / (float)K + sp.eps);
#pragma unroll
      for (int k = 0; k < kIter; ++k) {
        float f[8], w[8];
        unpack8(xreg[k], f);
        unpack8(wreg[k], w);
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] = round_bf16(f[j] * inv) * w[j];
        xreg[k] = pack8(f);
      }
    }
#pragma unroll
    for (int k = 0; k < kIter; ++k) {
      const int i = tid + k * kStepThreads;
      if (i < nch) xs[i] = xreg[k];
    }
  } else {
    // the attention phase left (D outputs, maximum, sum) per head and key split: fold them
    const int D = sp.D, ns = sp.nsplit, PS = D + 4;
    for (int i = tid; i < nch; i += kStepThreads) {
      const int h = (i * 8) / D, d0 = (i * 8) - h * D;
      const float* src = sp.att_part + (size_t)h * ns * PS;
      float ms[16], M = -INFINITY;
#pragma unroll
      for (int s = 0; s < 16; ++s) {
        ms[s] = s < ns ? __ldcg(src + s * PS + D) : -INFINITY;
        M = fmaxf(M, ms[s]);
      }
      float L = 0.f, acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll 4
      for (int s = 0; s < ns; ++s) {
        const float ls = __ldcg(src + s * PS + D + 1);
        const float4 o0 = __ldcg(reinterpret_cast<const float4*>(src + s * PS + d0));
        const float4 o1 = __ldcg(reinterpret_cast<const float4*>(src + s * PS + d0 + 4));
        const float mv = __ldcg(src + s * PS + D);
        const float c = (mv == -INFINITY) ? 0.f : exp2f(mv - M);
        L = fmaf(ls, c, L);
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
  step_stamp(sp, epoch, 1);

  // ---- this warp's items of the phase ----
  // A lane owns columns 8 * lane .. + 8 of the item; acc[r] holds the (even, odd) column
  // sums of row r as one packed pair.
  float2 acc[kItemRows];
#pragma unroll
  for (int r = 0; r < kItemRows; ++r) acc[r] = make_float2(0.f, 0.f);
  while (!st.con.done && st.con.pid == pid) {
    const Cursor& c = st.con;
    if (!ring_wait(st, c.idx, sp.status, &sh.abort)) break;
    const ItemGeom g = item_geom(c.ph, c.unit, c.item);
    if (lane * 8 < g.ncols) {
      const uint4* w = reinterpret_cast<const uint4*>(ring_bytes + (size_t)(c.idx % kSlots) * kSlotBytes) + lane;
      const uint4 xv = xs[(g.col0 >> 3) + lane];
      const float2 x0 = step_pair(xv.x), x1 = step_pair(xv.y), x2 = step_pair(xv.z), x3 = step_pair(xv.w);
#pragma unroll
      for (int r = 0; r < kItemRows; ++r) {
        const uint4 wv = w[r * (kRowPitch / 16)];
        acc[r] = __ffma2_rn(step_pair(wv.x), x0, acc[r]);
        acc[r] = __ffma2_rn(step_pair(wv.y), x1, acc[r]);
        acc[r] = __ffma2_rn(step_pair(wv.z), x2, acc[r]);
        acc[r] = __ffma2_rn(step_pair(wv.w), x3, acc[r]);
      }
    }
    // the slot is free: start the copy of the item kSlots ahead in the sequence
    __syncwarp();
    if (!st.iss.done) {
      if (lane == 0) ring_issue(st);
      cursor_advance(st.iss, sp, st.gw, st.NW);
    }
    if (c.item == c.ph.nitems - 1) {
      // Sum over the lanes and transpose in one pass: each exchange halves the rows a lane
      // still carries, so 8 rows x 32 lanes take 9 shuffles; lane L ends with row L / 4.
      float v[kItemRows];
#pragma unroll
      for (int r = 0; r < kItemRows; ++r) { v[r] = acc[r].x + acc[r].y; acc[r] = make_float2(0.f, 0.f); }
      float w4[4], w2[2], tot;
      {
        const bool up = lane & 16;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float send = up ? v[i] : v[i + 4], keep = up ? v[i + 4] : v[i];
          w4[i] = keep + __shfl_xor_sync(0xffffffffu, send, 16);
        }
      }
      {
        const bool up = lane & 8;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const float send = up ? w4[i] : w4[i + 2], keep = up ? w4[i + 2] : w4[i];
          w2[i] = keep + __shfl_xor_sync(0xffffffffu, send, 8);
        }
      }
      {
        const bool up = lane & 4;
        const float send = up ? w2[0] : w2[1], keep = up ? w2[1] : w2[0];
        tot = keep + __shfl_xor_sync(0xffffffffu, send, 4);
      }
      tot += __shfl_xor_sync(0xffffffffu, tot, 2);
      tot += __shfl_xor_sync(0xffffffffu, tot, 1);
      const int r = lane >> 2;
      if (c.ph.mode == PH_SWIGLU) {
        // rows 0-3 are gate rows (lanes 0-15), rows 4-7 the matching up rows (lanes 16-31)
        const float upv = __shfl_xor_sync(0xffffffffu, tot, 16);
        if (lane < 16 && (lane & 3) == 0) {
          const float act = round_bf16(silu_f32(round_bf16(tot)));
          a.y[g.group * 4 + r] = __float2bfloat16_rn(__fmul_rn(act, round_bf16(upv)));
        }
      } else if ((lane & 3) == 0) {
        const int row = g.group * kItemRows + r;
        if (c.ph.mode == PH_PART) {
          c.ph.part[(size_t)g.kpart * c.ph.rows + row] = tot;
        } else {
          const float lg = round_bf16(tot);
          a.y[row] = __float2bfloat16_rn(lg);
          best = step_max(best, step_key(lg, row));
        }
      }
    }
    cursor_advance(st.con, sp, st.gw, st.NW);
  }
  step_stamp(sp, epoch, 2);
  grid_arrive(sp.barrier);
  ++epoch;
  return true;
}

// One-query attention of every head over the cache rows [lo, pos], the keys of a head
// split over `nsplit` CTAs.  A unit is (head, split); the CTA leaves the unnormalised
// partial (D outputs, running maximum, sum) in sp.att_part for the o_proj phase to fold.
//
// This phase is also the consumer of the q/k/v projection: it sums that projection's K
// parts for its own query head and KV head, rounds to bf16 and applies RoPE to q and k
// (rows i and i + D/2 rotate together, cos at even and sin at odd columns of the angle
// row), and one CTA per KV head stores the new k and v rows into the caches.  The first
// batch of older K and V rows is in flight before the wait for the projection.
template <int D>
__device__ __forceinline__ bool attention_phase(const StepParams& sp, __nv_bfloat16* Kc, __nv_bfloat16* Vc,
                                                int pos, StepShared& sh, float (*sm_o)[D],
                                                unsigned int& epoch) {
  constexpr int LPK = D / 8, KPW = 32 / LPK, TS = KPW * kStepWarps, UNR = 4;
  constexpr int PS = D + 4, HALF = D / 2;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int dsel = lane % LPK, kslot = warp * KPW + lane / LPK;
  const int ns = sp.nsplit, units = sp.H * ns, group = sp.H / sp.G;
  const int kv_valid = pos + 1;
  const int lo = (sp.window >= 0) ? max(0, kv_valid - 1 - sp.window) : 0;
  const int per = (kv_valid - lo + ns - 1) / ns;
  const size_t row = (size_t)sp.G * D;   // elements between cache rows
  const int rows_qkv = (sp.H + 2 * sp.G) * D;

  int unit = blockIdx.x;
  int h = 0, split = 0, k_begin = 0, k_end = 0;
  const __nv_bfloat16 *Kb = Kc, *Vb = Vc;
  auto place = [&](int u) {
    h = u / ns;
    split = u - h * ns;
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
    if (early) load_batch(k_begin);   // the newest row is not in the cache yet: replaced below
  }
  // the RoPE row of this position
  float cs = 1.f, sn = 0.f;
  if (tid < 2 * HALF) {
    const int i = tid < HALF ? tid : tid - HALF;
    const __nv_bfloat16* ang = sp.angles + (size_t)pos * D;
    cs = __bfloat162float(ang[2 * i]);
    sn = __bfloat162float(ang[2 * i + 1]);
  }

  if (!grid_wait(sp.barrier, epoch, sp.status, &sh.abort)) return false;
  step_stamp(sp, epoch, 0);
  step_stamp(sp, epoch, 1);

  for (; unit < units; unit += gridDim.x) {
    if (!early) place(unit);
    // ---- q, and the new k and v rows of this head's KV head, from the projection's parts ----
    {
      const int kh = h / group;
      auto part_sum = [&](int r) {
        float s = 0.f;
        for (int p = 0; p < sp.kp_qkv; ++p) s += __ldcg(sp.part_qkv + (size_t)p * rows_qkv + r);
        return round_bf16(s);
      };
      if (tid < 2 * HALF) {
        // threads [0, HALF): q pairs; [HALF, 2 HALF): k pairs
        const bool is_k = tid >= HALF;
        const int i = is_k ? tid - HALF : tid;
        const int base = is_k ? (sp.H + kh) * D : h * D;
        const float x1 = part_sum(base + i), x2 = part_sum(base + i + HALF);
        const float y1 = round_bf16(__fsub_rn(__fmul_rn(x1, cs), __fmul_rn(x2, sn)));
        const float y2 = round_bf16(__fadd_rn(__fmul_rn(x2, cs), __fmul_rn(x1, sn)));
        if (is_k) {
          sh.knew[i] = __float2bfloat16_rn(y1);
          sh.knew[i + HALF] = __float2bfloat16_rn(y2);
        } else {
          sh.q[i] = y1 * sp.scale_log2;
          sh.q[i + HALF] = y2 * sp.scale_log2;
        }
      }
      if (tid >= kStepThreads - D) {
        const int i = tid - (kStepThreads - D);
        sh.vnew[i] = __float2bfloat16_rn(part_sum((sp.H + sp.G + kh) * D + i));
      }
      __syncthreads();
      if (h == kh * group && split == 0 && tid < 2 * LPK) {
        // one CTA per KV head stores the new rows for the steps to come
        const int i = tid % LPK;
        __nv_bfloat16* dst = (tid < LPK ? Kc : Vc) + (size_t)pos * row + (size_t)kh * D + i * 8;
        *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>((tid < LPK ? sh.knew : sh.vnew) + i * 8);
      }
    }
    float q[8], o[8], m = -INFINITY, l = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) { q[j] = sh.q[dsel * 8 + j]; o[j] = 0.f; }
    for (int kb = k_begin; kb < k_end; kb += TS * UNR) {
      if (!(early && kb == k_begin)) load_batch(kb);
      // the newest row comes from this step's projection
#pragma unroll
      for (int u = 0; u < UNR; ++u) {
        if (kb + u * TS + kslot == kv_valid - 1) {
          kraw[u] = *reinterpret_cast<const uint4*>(sh.knew + dsel * 8);
          vraw[u] = *reinterpret_cast<const uint4*>(sh.vnew + dsel * 8);
        }
      }
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
  step_stamp(sp, epoch, 2);
  grid_arrive(sp.barrier);
  ++epoch;
  return true;
}

template <int D>
__global__ void __launch_bounds__(kStepThreads, 1) decode_step_kernel(const StepParams sp) {
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ StepShared sh;
  __shared__ __align__(16) float sm_o[kStepWarps][D];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  unsigned char* xs_bytes = smem + kStepRingBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kStepBarsOff);
  for (int i = tid; i < sp.L * 9; i += kStepThreads)
    reinterpret_cast<const void**>(layer_table())[i] = reinterpret_cast<const void* const*>(sp.layers)[i];
  if (tid == 0) {
    sh.abort = 0;
    for (int i = 0; i < kStepWarps * kSlots; ++i) step_mbar_init(bars + i, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  // ---- start the weight stream: the first kSlots items of this warp's sequence ----
  Stream st;
  st.slots = smem_u32(smem) + (uint32_t)(warp * kSlots * kSlotBytes);
  st.bars = bars + warp * kSlots;
  st.policy = step_evict_first_policy();
  st.NW = gridDim.x * kStepWarps;
  st.gw = warp * gridDim.x + blockIdx.x;   // neighbouring units go to different SMs
  cursor_start(st.con, sp, st.gw, st.NW);
  st.iss = st.con;
  for (int i = 0; i < kSlots && !st.iss.done; ++i) {
    if (lane == 0) ring_issue(st);
    cursor_advance(st.iss, sp, st.gw, st.NW);
  }

  // (token, position) were left by the previous step or by the host
  int token = sp.values[0], pos = sp.values[1];
  token = max(0, min(token, sp.V - 1));
  pos = max(0, min(pos, sp.S - 1));
  unsigned int epoch = 0;
  unsigned long long best = 0ull;
  bool ok = true;
  const __nv_bfloat16* x0 = sp.embed + (size_t)token * sp.E;   // layer 0's residual stream

  // One loop over the step's phases with one call site per kind of phase keeps the code of
  // the whole step small enough for the instruction cache.
  const int phases = 5 * sp.L + 1;
#pragma unroll 1
  for (int p = 0; p < phases && ok; ++p) {
    const int l = p / 5, j = p - 5 * l;
    const StepLayer& ly = layer_table()[l < sp.L ? l : 0];
    if (l < sp.L && j == 1) {
      ok = attention_phase<D>(sp, ly.k, ly.v, pos, sh, sm_o, epoch);
      continue;
    }
    PhaseArgs a = {};
    int pid;
    if (l >= sp.L || j == 0) {
      // the residual stream after the layer before (or the embedding row), then the final
      // norm and the head, or this layer's first norm and q/k/v
      if (l == 0) {
        a.stage = ST_VECTOR; a.x = x0;
      } else {
        a.stage = ST_PARTIAL; a.parts = sp.part_d; a.nparts = sp.kp_d; a.residual = sp.xb; a.keep = sp.xa;
      }
      a.K = sp.E;
      if (l >= sp.L) { a.mode = PH_HEAD; pid = 4 * sp.L; a.norm_w = sp.final_norm; a.y = sp.logits; }
      else { a.mode = PH_PART; pid = 4 * l; a.norm_w = ly.ln1; }
    } else if (j == 2) {      // attention fold, o_proj
      a.mode = PH_PART; pid = 4 * l + 1; a.stage = ST_ATTENTION; a.K = sp.H * D;
    } else if (j == 3) {      // residual, RMSNorm, gate/up, SiLU, product
      a.mode = PH_SWIGLU; pid = 4 * l + 2; a.stage = ST_PARTIAL; a.K = sp.E;
      a.parts = sp.part_o; a.nparts = sp.kp_o; a.residual = l == 0 ? x0 : sp.xa; a.keep = sp.xb;
      a.norm_w = ly.ln2; a.y = sp.act;
    } else {                  // down_proj
      a.mode = PH_PART; pid = 4 * l + 3; a.stage = ST_VECTOR; a.x = sp.act; a.K = sp.F;
    }
    ok = weight_phase(sp, pid, a, st, smem + (size_t)warp * kSlots * kSlotBytes, xs_bytes, sh, epoch, best);
  }
  if (!ok || sh.abort) {
    // the step is abandoned: let this warp's copies in flight land before the CTA leaves
    const unsigned long long t0 = step_ns();
    for (int idx = st.con.idx; idx < st.iss.idx; ++idx) {
      uint64_t* bar = st.bars + idx % kSlots;
      const uint32_t parity = (uint32_t)(idx / kSlots) & 1u;
      while (!step_mbar_try_wait(bar, parity) && step_ns() - t0 < kStepWaitNs) {}
    }
    return;
  }
  // ---- greedy draw: CTA maxima, then CTA 0 folds them ----
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

// K parts of a narrow projection: the smallest power of two that gives the grid's warps a
// unit each, while a part keeps whole 32-column blocks.
static int pick_parts(int rows, int K, int warps) {
  int p = 1;
  while (p < kStepMaxParts && (rows / kItemRows) * p * 5 < warps * 4 && K % (2 * p * kItemCols) == 0) p *= 2;
  return p;
}

// ---- tensor maps of the weight matrices (host) ----------------------------------------
typedef CUresult (*StepEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                 const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                 CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static StepEncodeFn step_encode_fn() {
  static StepEncodeFn fn = [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      return reinterpret_cast<StepEncodeFn>(sym);
    return static_cast<StepEncodeFn>(nullptr);
  }();
  return fn;
}
// A (rows, K) row-major bf16 matrix, read in boxes of `box_rows` rows x 256 columns.
static bool step_make_map(CUtensorMap* map, const void* base, int rows, int K, int box_rows) {
  StepEncodeFn fn = step_encode_fn();
  if (!fn) return false;
  const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
  const cuuint32_t box[2] = {(cuuint32_t)kItemCols, (cuuint32_t)box_rows};
  const cuuint32_t elem[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int D>
static int launch_step(StepParams& sp, cudaStream_t stream) {
  static int grid = 0;
  if (grid == 0) {
    if (cudaFuncSetAttribute(decode_step_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)kStepSmem) != cudaSuccess)
      return IRON_ERR_LAUNCH;
    int per_sm = 0, dev = 0, sms = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_step_kernel<D>, kStepThreads, kStepSmem) !=
            cudaSuccess ||
        cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
      return IRON_ERR_LAUNCH;
    if (per_sm < 1 || sms < 1) return IRON_ERR_LAUNCH;
    grid = sms > 512 ? 512 : sms;
  }
  const int warps = grid * kStepWarps;
  sp.kp_qkv = pick_parts((sp.H + 2 * sp.G) * sp.D, sp.E, warps);
  sp.kp_o = pick_parts(sp.E, sp.H * sp.D, warps);
  sp.kp_d = pick_parts(sp.E, sp.F, warps);
  // keys of a head go to as many CTAs as the grid has per head
  int ns = grid / sp.H;
  sp.nsplit = ns < 1 ? 1 : (ns > 16 ? 16 : ns);
  if (cudaMemsetAsync(sp.barrier, 0, sizeof(unsigned int), stream) != cudaSuccess) return IRON_ERR_LAUNCH;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid, 1, 1);
  cfg.blockDim = dim3(kStepThreads, 1, 1);
  cfg.dynamicSmemBytes = kStepSmem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;   // every CTA resident: the barrier cannot starve
  attr[0].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (cudaLaunchKernelEx(&cfg, decode_step_kernel<D>, sp) != cudaSuccess) return IRON_ERR_LAUNCH;
  return IRON_OK;
}

// Workspace layout (bytes): barrier word at 0, status word at 128, one key per CTA at 256,
// then the attention partials, the trace and the three projections' f32 partial sums.
struct StepWorkspace {
  size_t best, att, trace, part_qkv, part_o, part_d, total;
};
static StepWorkspace step_workspace(int E, int H, int G, int D) {
  StepWorkspace w;
  w.best = 256;
  w.att = w.best + 512 * sizeof(unsigned long long);
  w.trace = w.att + (size_t)H * 16 * (D + 4) * sizeof(float);
  w.part_qkv = w.trace + 1024 * sizeof(unsigned long long);
  w.part_o = w.part_qkv + (size_t)kStepMaxParts * (H + 2 * G) * D * sizeof(float);
  w.part_d = w.part_o + (size_t)kStepMaxParts * E * sizeof(float);
  w.total = w.part_d + (size_t)kStepMaxParts * E * sizeof(float);
  return w;
}

}  // namespace iron

using namespace iron;

extern "C" size_t iron_decode_step_workspace_bytes(int E, int H, int G, int D) {
  if (E <= 0 || H <= 0 || G <= 0 || D <= 0) return 0;
  return step_workspace(E, H, G, D).total;
}

extern "C" size_t iron_decode_step_maps_bytes(int L) {
  return L > 0 ? (size_t)(kMapsPerLayer * L + 1) * sizeof(CUtensorMap) : 0;
}

extern "C" int iron_decode_step_encode_maps(const void* const* h_layer_ptrs, int L, int E, int F, int H, int G,
                                            int D, int V, const void* head, void* h_maps_out) {
  if (!h_layer_ptrs || !h_maps_out || !head) return IRON_ERR_SHAPE;
  if (L <= 0 || L > kStepMaxLayers || E <= 0 || F <= 0 || H <= 0 || G <= 0 || D <= 0 || V <= 0) return IRON_ERR_SHAPE;
  if ((E & 31) || (F & 31) || ((H * D) & 31)) return IRON_ERR_SHAPE;
  CUtensorMap* out = static_cast<CUtensorMap*>(h_maps_out);
  for (int l = 0; l < L; ++l) {
    const void* const* p = h_layer_ptrs + 9 * l;   // ln1, wqkv, wo, ln2, wg, wu, wd, k, v
    for (int i = 0; i < 9; ++i)
      if (!p[i] || (reinterpret_cast<uintptr_t>(p[i]) & 15u)) return IRON_ERR_ALIGN;
    CUtensorMap* m = out + kMapsPerLayer * l;
    if (!step_make_map(m + 0, p[1], (H + 2 * G) * D, E, kItemRows) ||
        !step_make_map(m + 1, p[2], E, H * D, kItemRows) ||
        !step_make_map(m + 2, p[4], F, E, 4) ||
        !step_make_map(m + 3, p[5], F, E, 4) ||
        !step_make_map(m + 4, p[6], E, F, kItemRows))
      return IRON_ERR_LAUNCH;
  }
  if (reinterpret_cast<uintptr_t>(head) & 15u) return IRON_ERR_ALIGN;
  if (!step_make_map(out + kMapsPerLayer * L, head, V, E, kItemRows)) return IRON_ERR_LAUNCH;
  return IRON_OK;
}

extern "C" int iron_decode_step_bf16(const void* const* layer_ptrs, const void* maps, int L, int E, int F, int H, int G,
                                     int D, int V, int S, const void* embed, const void* head,
                                     const void* final_norm, const void* angles, float eps,
                                     float scale, int window, int* values, int* drawn, void* xa,
                                     void* xb, void* act, void* logits, void* workspace,
                                     iron_stream_t stream) {
  if (L <= 0 || E <= 0 || F <= 0 || H <= 0 || G <= 0 || V <= 0 || S <= 0 || H % G) return IRON_ERR_SHAPE;
  if (D != 64 && D != 128) return IRON_ERR_SHAPE;
  if (L > kStepMaxLayers) return IRON_ERR_SHAPE;
  if ((E & 31) || (F & 31) || ((H * D) & 31) || (V & 7) || (F & 3)) return IRON_ERR_SHAPE;
  if (E > kStepMaxK || F > kStepMaxK || H * D > kStepMaxK) return IRON_ERR_SHAPE;
  const void* must16[] = {embed, head, xa, xb, act, logits, workspace, final_norm, angles};
  for (const void* p : must16)
    if (!p || (reinterpret_cast<uintptr_t>(p) & 15u)) return IRON_ERR_ALIGN;
  if (!layer_ptrs || !maps || !values || !drawn) return IRON_ERR_SHAPE;
  if (reinterpret_cast<uintptr_t>(maps) & 63u) return IRON_ERR_ALIGN;
  StepParams sp = {};
  sp.layers = reinterpret_cast<const StepLayer*>(layer_ptrs);
  sp.maps = static_cast<const CUtensorMap*>(maps);
  sp.L = L; sp.E = E; sp.F = F; sp.H = H; sp.G = G; sp.D = D; sp.V = V; sp.S = S;
  sp.embed = (const __nv_bfloat16*)embed; sp.head = (const __nv_bfloat16*)head;
  sp.final_norm = (const __nv_bfloat16*)final_norm; sp.angles = (const __nv_bfloat16*)angles;
  sp.eps = eps; sp.scale_log2 = scale * 1.4426950408889634f; sp.window = window;
  sp.values = values; sp.drawn = drawn;
  sp.xa = (__nv_bfloat16*)xa; sp.xb = (__nv_bfloat16*)xb;
  sp.act = (__nv_bfloat16*)act; sp.logits = (__nv_bfloat16*)logits;
  const StepWorkspace w = step_workspace(E, H, G, D);
  char* ws = static_cast<char*>(workspace);
  sp.barrier = reinterpret_cast<unsigned int*>(ws);
  sp.status = reinterpret_cast<int*>(ws + 128);
  sp.best = reinterpret_cast<unsigned long long*>(ws + w.best);
  sp.att_part = reinterpret_cast<float*>(ws + w.att);
  sp.trace = reinterpret_cast<unsigned long long*>(ws + w.trace);
  sp.part_qkv = reinterpret_cast<float*>(ws + w.part_qkv);
  sp.part_o = reinterpret_cast<float*>(ws + w.part_o);
  sp.part_d = reinterpret_cast<float*>(ws + w.part_d);
  return D == 64 ? launch_step<64>(sp, (cudaStream_t)stream) : launch_step<128>(sp, (cudaStream_t)stream);
}
