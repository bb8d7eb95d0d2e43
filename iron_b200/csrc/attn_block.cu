// One decode step's attention and o_proj of a Llama-style layer in ONE kernel:
//
//     y = x + Wo . attention(q, cache keys 0 .. position, cache values 0 .. position)
//
// i.e. the reference's steps MHA, o_proj and the residual add (iron/lm/blocks.py:487-502,
// :646-648, :723-728) -- two dependent launches of the separate-kernel path (split-K
// attention, o_proj GEMV), each a few microseconds of launch-to-launch latency for 4-8 MB.
// Only the final sum needs the whole GPU to agree, because the work splits by KV group: the
// query heads of group g read only the keys and values of group g, and their share of
// o_proj is the 'QH * D' columns of Wo that multiply their outputs.
//
// A thread-block cluster of eight CTAs owns one KV group.  Its CTAs
//   1. (before the dependency wait, i.e. while the q/k/v projection kernel still runs) start
//      every byte they will need on its way into shared memory: their 'E / 8' rows of the
//      group's column block of Wo by bulk copies (cp.async.bulk + mbarrier) and their eighth
//      of the group's cached keys and values by 16-byte asynchronous copies -- everything but
//      the newest cache row, which the projection kernel is still writing;
//   2. wait for that kernel, read q and the newest k/v row, and run the one-query attention
//      of the group's heads over their keys in three passes that have no loop-carried
//      dependency (all scores; maximum, exponentials and sum per head; the weighted sum of
//      values), so the passes are bound by issue rate, not by a chain of latencies;
//   3. (cluster barrier) merge the eight (max, sum, output) partials over distributed shared
//      memory -- every CTA then holds the group's attention output, rounded to bf16 as the
//      MHA operator's output is;
//   4. multiply their rows of Wo's column block by it, one row per thread out of shared
//      memory: a float32 partial of y per group, written to a scratch the caller provides.
// For every eighth of y's rows the last of the CTAs holding it (an arrival counter per
// eighth; nobody waits for anybody) adds the G partials in group order, rounds as the o_proj
// GEMV's output rounds, adds the residual and rounds again.  The wait on the bulk copies is
// bounded; if it gives up the kernel records IRON_ERR_TIMEOUT and walks on through the same
// barriers, so a lost copy costs a wrong vector and an error status, never a hang.
#include <cooperative_groups.h>

#include "common.cuh"
#include "gemv_items.cuh"
#include "mma.cuh"

namespace cg = cooperative_groups;

namespace iron {

constexpr int kAbThreads = 256;
constexpr int kAbWarps = kAbThreads / 32;
constexpr int kAbCluster = 8;                              // CTAs per KV group
constexpr unsigned long long kAbWaitNs = 2000000000ull;    // 2 s

struct AttnBlockParams {
  const __nv_bfloat16* q;        // (H, D) rotated queries
  const __nv_bfloat16* wo;       // (E, H * D)
  const __nv_bfloat16* x;        // (E) the residual stream
  const __nv_bfloat16* k_cache;  // (cache_rows, G, D)
  const __nv_bfloat16* v_cache;
  __nv_bfloat16* y;              // (E)
  float* partial;                // (G, E) scratch
  unsigned int* counters;        // kAbCluster words, zero between launches
  const int* d_position;
  int position;
  int E, H, G, cache_rows, window, kcap;
  float scale_log2;
  int* status;
  unsigned long long* trace;     // optional: 16 timestamps (ns) per CTA, a diagnostic
};

__device__ __forceinline__ void ab_mbar_init(uint64_t* bar) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void ab_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool ab_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}
__device__ __forceinline__ void ab_bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar,
                                             uint64_t policy) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
      ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)), "l"(policy) : "memory");
}
__device__ __forceinline__ unsigned long long ab_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
// Wait for phase 0 of `bar`; false when the limit ran out.
__device__ __forceinline__ bool ab_wait(uint64_t* bar) {
  if (ab_try_wait(bar, 0)) return true;
  unsigned long long t0 = 0;
  for (uint32_t it = 1; !ab_try_wait(bar, 0); ++it) {
    if ((it & 255u) != 0) continue;
    const unsigned long long now = ab_ns();
    if (t0 == 0) t0 = now;
    else if (now - t0 > kAbWaitNs) return false;
  }
  return true;
}
__device__ __forceinline__ void ab_cp16(void* dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void ab_cp_wait_all() {
  asm volatile("cp.async.commit_group;\n\tcp.async.wait_group 0;" ::: "memory");
}
__device__ __forceinline__ void ab_cluster_arrive() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
}
__device__ __forceinline__ void ab_cluster_wait() {
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// Shared-memory plan of one CTA (bytes).  Rows of keys, values and Wo are padded by 16 bytes
// so that threads walking down a column of 16-byte chunks hit different banks.
struct AbLayout {
  int wo_rows, wo_cols, wo_pitch, kv_pitch;   // pitches in elements
  size_t off_wo, off_k, off_v, off_q, off_sc, off_part, off_att, off_pv, off_misc, total;
};
__host__ __device__ inline AbLayout ab_layout(int D, int QH, int E, int kcap) {
  AbLayout L;
  L.wo_rows = E / kAbCluster;
  L.wo_cols = QH * D;
  L.wo_pitch = L.wo_cols + 8;
  L.kv_pitch = D + 8;
  size_t o = 0;
  auto take = [&o](size_t bytes) { const size_t at = o; o += (bytes + 15) & ~(size_t)15; return at; };
  L.off_wo = take((size_t)L.wo_rows * L.wo_pitch * 2);
  L.off_k = take((size_t)kcap * L.kv_pitch * 2);
  L.off_v = take((size_t)kcap * L.kv_pitch * 2);
  L.off_q = take((size_t)QH * D * 2);
  L.off_sc = take((size_t)QH * kcap * 4);               // scores, then probabilities
  L.off_part = take((size_t)QH * (D + 2) * 4);          // this CTA's (output, max, sum) per head
  L.off_att = take((size_t)QH * D * 2);
  L.off_pv = take((size_t)QH * D * 4);                  // a chunk's weighted sum of values
  L.off_misc = take(64 + 32 * 4);                       // one mbarrier and a flag, then max and sum per head
  L.total = o;
  return L;
}

#define AB_STAMP(i) do { if (p.trace && threadIdx.x == 0) p.trace[(size_t)blockIdx.x * 16 + (i)] = ab_ns(); } while (0)

template <int D, int QH>
__global__ void __launch_bounds__(kAbThreads, 2) attn_oproj_kernel(const AttnBlockParams p) {
  extern __shared__ __align__(128) unsigned char ab_smem[];
  AB_STAMP(0);
  cg::cluster_group cluster = cg::this_cluster();
  constexpr int NC = kAbCluster;
  constexpr int OUT = QH * D;                            // the group's attention output; <= kAbThreads
  const int c = (int)cluster.block_rank();
  const int g = blockIdx.x / NC;                         // KV group of this cluster
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int E = p.E;
  const AbLayout L = ab_layout(D, QH, E, p.kcap);
  __nv_bfloat16* wosm = reinterpret_cast<__nv_bfloat16*>(ab_smem + L.off_wo);
  __nv_bfloat16* ksm = reinterpret_cast<__nv_bfloat16*>(ab_smem + L.off_k);
  __nv_bfloat16* vsm = reinterpret_cast<__nv_bfloat16*>(ab_smem + L.off_v);
  __nv_bfloat16* qsm = reinterpret_cast<__nv_bfloat16*>(ab_smem + L.off_q);
  float* sc = reinterpret_cast<float*>(ab_smem + L.off_sc);              // [QH][kcap]
  float* part = reinterpret_cast<float*>(ab_smem + L.off_part);          // [QH][D + 2]
  __nv_bfloat16* att = reinterpret_cast<__nv_bfloat16*>(ab_smem + L.off_att);
  float* pv = reinterpret_cast<float*>(ab_smem + L.off_pv);              // [QH][D]
  uint64_t* bar = reinterpret_cast<uint64_t*>(ab_smem + L.off_misc);
  int* flags = reinterpret_cast<int*>(bar + 1);                          // [0] last of the row slice
  float* red = reinterpret_cast<float*>(ab_smem + L.off_misc + 64);      // [QH][2] max and sum per head

  if (tid == 0) {
    ab_mbar_init(bar);
    flags[0] = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  pdl_launch();

  // ---- 1. everything this CTA will read, on its way before the dependency resolves ----
  if (warp < 2) {
    uint64_t policy;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
    if (tid == 0) ab_expect_tx(bar, (uint32_t)L.wo_rows * (uint32_t)L.wo_cols * 2u);
    asm volatile("bar.sync 1, 64;" ::: "memory");        // the two issuing warps only
    const size_t pitch = (size_t)p.H * D;
    for (int r = tid; r < L.wo_rows; r += 64)
      ab_bulk_load(wosm + (size_t)r * L.wo_pitch, p.wo + (size_t)(c * L.wo_rows + r) * pitch + (size_t)g * L.wo_cols,
                   (uint32_t)L.wo_cols * 2u, bar, policy);
  }
  // The position was written by the draw of the previous step, kernels ago; it is read again
  // after the wait, and the keys are fetched again if it was not yet there.
  auto key_range = [&](int pos, int& kb, int& ke) {
    const int kv_valid = pos + 1;
    const int lo_all = (p.window >= 0) ? max(0, kv_valid - 1 - p.window) : 0;
    const int per = (kv_valid - lo_all + NC - 1) / NC;
    kb = lo_all + c * per;
    ke = min(kv_valid, kb + per);
  };
  auto fetch_keys = [&](int k0, int k1, int newest) {   // cache rows [k0, k1) but `newest` (< 0: none)
    const int n = k1 - k0;
    constexpr int CH = D / 8;
    for (int idx = tid; idx < n * CH; idx += kAbThreads) {
      const int j = idx / CH, ch = idx - j * CH;
      if (k0 + j == newest) continue;
      const size_t src = ((size_t)(k0 + j) * p.G + g) * D + ch * 8;
      ab_cp16(ksm + (size_t)j * L.kv_pitch + ch * 8, p.k_cache + src);
      ab_cp16(vsm + (size_t)j * L.kv_pitch + ch * 8, p.v_cache + src);
    }
  };
  const int pos_early = min(max(p.d_position ? *p.d_position : p.position, 0), p.cache_rows - 1);
  int kb, ke;
  key_range(pos_early, kb, ke);
  fetch_keys(kb, min(ke, kb + p.kcap), pos_early);
  AB_STAMP(1);

  pdl_wait();
  AB_STAMP(2);

  // ---- 2. q, the newest cache row, and the attention of the group's heads over this CTA's keys ----
  // q and the newest row are asked for at once, at the position read before the wait; the
  // position is read again beside them, and only if it changed are the keys fetched again
  if (tid < OUT / 8)
    reinterpret_cast<uint4*>(qsm)[tid] = ld_cached(reinterpret_cast<const uint4*>(p.q + (size_t)g * OUT) + tid);
  if (pos_early >= kb && pos_early < min(ke, kb + p.kcap)) {
    constexpr int CH = D / 8;
    if (tid >= 64 && tid < 64 + 2 * CH) {
      const int t2 = tid - 64, ch = t2 % CH;
      const size_t src = ((size_t)pos_early * p.G + g) * D + ch * 8;
      ab_cp16((t2 < CH ? ksm : vsm) + (size_t)(pos_early - kb) * L.kv_pitch + ch * 8,
              (t2 < CH ? p.k_cache : p.v_cache) + src);
    }
  }
  const int pos = min(max(p.d_position ? *p.d_position : p.position, 0), p.cache_rows - 1);
  key_range(pos, kb, ke);
  float m_run = -INFINITY, l_run = 0.f, o_run = 0.f;     // thread (h, d)'s running values across chunks
  const int oh = tid / D, od = tid - oh * D;             // pass 3: thread -> (head, output column)
  bool first = (pos == pos_early);
  for (int cs = kb; cs < ke; cs += p.kcap) {
    const int ce = min(ke, cs + p.kcap);
    const int n = ce - cs;
    if (!first) {   // a later chunk (or keys fetched for a stale position): the buffers are reused
      ab_cp_wait_all();
      __syncthreads();
      fetch_keys(cs, ce, -1);
    }
    first = false;
    ab_cp_wait_all();
    __syncthreads();
    {   // the value rows a 16-key tile reads past the chunk's last key must be numbers: zeros
      constexpr int CH = D / 8;
      const int pad = ((n + 15) & ~15) - n;
      for (int idx = tid; idx < pad * CH; idx += kAbThreads)
        *reinterpret_cast<uint4*>(vsm + (size_t)(n + idx / CH) * L.kv_pitch + (idx % CH) * 8) = make_uint4(0, 0, 0, 0);
    }
    // pass 1: every score of the chunk on the tensor cores: 16 keys x (heads padded to 8) per
    // warp tile, K rows as the A operand, q as the B operand (held in registers for all tiles)
    {
      const int gq = lane >> 2, tq = lane & 3;
      uint32_t bq[D / 16][2];
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks) {
        bq[ks][0] = gq < QH ? *reinterpret_cast<const uint32_t*>(qsm + gq * D + ks * 16 + 2 * tq) : 0u;
        bq[ks][1] = gq < QH ? *reinterpret_cast<const uint32_t*>(qsm + gq * D + ks * 16 + 8 + 2 * tq) : 0u;
      }
      for (int j0 = warp * 16; j0 < n; j0 += kAbWarps * 16) {   // rows past n hold stale keys: not stored
        float cacc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
          uint32_t a[4];
          load_a_rowmajor(a, ksm, L.kv_pitch, j0, ks * 16, lane);
          mma_bf16_16816(cacc, a, bq[ks][0], bq[ks][1]);
        }
        if (2 * tq < QH) {
          const int ja = j0 + gq, jb = j0 + gq + 8;
          if (ja < n) {
            sc[(2 * tq) * p.kcap + ja] = cacc[0] * p.scale_log2;
            if (2 * tq + 1 < QH) sc[(2 * tq + 1) * p.kcap + ja] = cacc[1] * p.scale_log2;
          }
          if (jb < n) {
            sc[(2 * tq) * p.kcap + jb] = cacc[2] * p.scale_log2;
            if (2 * tq + 1 < QH) sc[(2 * tq + 1) * p.kcap + jb] = cacc[3] * p.scale_log2;
          }
        }
      }
    }
    __syncthreads();
    // pass 2: per head (one warp each) the chunk's maximum, the exponentials and their sum
    if (warp < QH) {
      float* s = sc + warp * p.kcap;
      float mx = -INFINITY;
      for (int j = lane; j < n; j += 32) mx = fmaxf(mx, s[j]);
      mx = warp_max(mx);
      float sum = 0.f;
      for (int j = lane; j < n; j += 32) {
        const float e = exp2f(s[j] - mx);
        s[j] = e;
        sum += e;
      }
      sum = warp_sum(sum);
      if (lane == 0) { red[warp * 2] = mx; red[warp * 2 + 1] = sum; }
    }
    __syncthreads();
    // pass 3: the weighted sum of values on the tensor cores: the probabilities (heads padded
    // to 16 rows, rounded to bf16) as the A operand, V rows as the B operand; a warp owns the
    // output columns [wcol0, wcol0 + 16) over all keys of the chunk
    for (int wcol0 = warp * 16; wcol0 < D; wcol0 += kAbWarps * 16) {
      const int gq = lane >> 2, tq = lane & 3;
      float c0[4] = {0.f, 0.f, 0.f, 0.f}, c1[4] = {0.f, 0.f, 0.f, 0.f};
      const float* pr = sc + gq * p.kcap;
      for (int j0 = 0; j0 < n; j0 += 16) {
        // a probability is split into a bf16 head and a bf16 remainder (two products), so the
        // weighted sum keeps float32's accuracy as the one-query kernel's does
        uint32_t a[4] = {0u, 0u, 0u, 0u}, r[4] = {0u, 0u, 0u, 0u};
        if (gq < QH) {   // keys past n contribute nothing
          const int ja = j0 + 2 * tq, jb = ja + 8;
          const float p0 = ja < n ? pr[ja] : 0.f, p1 = ja + 1 < n ? pr[ja + 1] : 0.f;
          const float p2 = jb < n ? pr[jb] : 0.f, p3 = jb + 1 < n ? pr[jb + 1] : 0.f;
          a[0] = pack_bf16x2(p0, p1);
          a[2] = pack_bf16x2(p2, p3);
          r[0] = pack_bf16x2(p0 - bf16_lo(a[0]), p1 - bf16_hi(a[0]));
          r[2] = pack_bf16x2(p2 - bf16_lo(a[2]), p3 - bf16_hi(a[2]));
        }
        uint32_t b[4];
        load_b_kn(b, vsm, L.kv_pitch, wcol0, j0, lane);
        mma_bf16_16816(c0, a, b[0], b[1]);
        mma_bf16_16816(c1, a, b[2], b[3]);
        mma_bf16_16816(c0, r, b[0], b[1]);
        mma_bf16_16816(c1, r, b[2], b[3]);
      }
      if (gq < QH) {   // rows of the tile are heads: c[0], c[1] are (head gq, columns 2 tq, 2 tq + 1)
        float* dst = pv + gq * D + wcol0 + 2 * tq;
        dst[0] = c0[0]; dst[1] = c0[1];
        dst[8] = c1[0]; dst[9] = c1[1];
      }
    }
    __syncthreads();
    if (tid < OUT) {
      const float acc = pv[oh * D + od];
      const float mc = red[oh * 2], lc = red[oh * 2 + 1];
      const float mn = fmaxf(m_run, mc);
      const float ca = (m_run == -INFINITY) ? 0.f : exp2f(m_run - mn);
      const float cb = exp2f(mc - mn);
      o_run = o_run * ca + acc * cb;
      l_run = l_run * ca + lc * cb;
      m_run = mn;
    }
  }
  if (tid < OUT) {
    part[oh * (D + 2) + od] = o_run;
    if (od == 0) { part[oh * (D + 2) + D] = m_run; part[oh * (D + 2) + D + 1] = l_run; }
  }
  AB_STAMP(3);
  cluster.sync();
  AB_STAMP(4);

  // ---- 3. fold the cluster's partials: every CTA needs the whole output for its rows of Wo ----
  if (tid < OUT) {
    float mr[NC], lr[NC], orr[NC];
#pragma unroll
    for (int r = 0; r < NC; ++r) {
      const float* remote = cluster.map_shared_rank(part, r);
      mr[r] = remote[oh * (D + 2) + D];
      lr[r] = remote[oh * (D + 2) + D + 1];
      orr[r] = remote[oh * (D + 2) + od];
    }
    float M = -INFINITY;
#pragma unroll
    for (int r = 0; r < NC; ++r) M = fmaxf(M, mr[r]);
    float Ls = 0.f, acc = 0.f;
#pragma unroll
    for (int r = 0; r < NC; ++r) {
      const float cf = (mr[r] == -INFINITY) ? 0.f : exp2f(mr[r] - M);
      Ls = fmaf(lr[r], cf, Ls);
      acc = fmaf(orr[r], cf, acc);
    }
    att[tid] = __float2bfloat16_rn(Ls > 0.f ? acc / Ls : 0.f);
  }
  ab_cluster_arrive();     // this CTA no longer reads its peers' shared memory (waited for at the end)
  __syncthreads();
  AB_STAMP(5);

  // ---- 4. this CTA's rows of Wo's column block times the group's output: a row per thread ----
  const bool ok = ab_wait(bar);
  AB_STAMP(6);
  {
    // 16 rows of Wo per warp tile as the A operand; the B operand's only live column is the
    // group's output (lanes of column 0 hold it, the rest zeros), kept in registers
    const int gq = lane >> 2, tq = lane & 3;
    uint32_t bo[OUT / 16][2];
#pragma unroll
    for (int ks = 0; ks < OUT / 16; ++ks) {
      bo[ks][0] = gq == 0 ? *reinterpret_cast<const uint32_t*>(att + ks * 16 + 2 * tq) : 0u;
      bo[ks][1] = gq == 0 ? *reinterpret_cast<const uint32_t*>(att + ks * 16 + 8 + 2 * tq) : 0u;
    }
    for (int r0 = warp * 16; r0 < L.wo_rows; r0 += kAbWarps * 16) {
      float cacc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int ks = 0; ks < OUT / 16; ++ks) {
        uint32_t a[4];
        load_a_rowmajor(a, wosm, L.wo_pitch, r0, ks * 16, lane);
        mma_bf16_16816(cacc, a, bo[ks][0], bo[ks][1]);
      }
      if (tq == 0) {   // column 0: rows r0 + gq and r0 + gq + 8
        float* dst = p.partial + (size_t)g * E + c * L.wo_rows + r0 + gq;
        dst[0] = cacc[0];
        dst[8] = cacc[2];
      }
    }
  }
  if (!ok && tid == 0 && p.status) *reinterpret_cast<volatile int*>(p.status) = IRON_ERR_TIMEOUT;
  AB_STAMP(7);
  // the CTAs (one per group) holding row slice `c`: the last to arrive sums it
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const unsigned int arrived = atomicAdd(p.counters + c, 1u);
    flags[0] = arrived == (unsigned int)p.G - 1;
  }
  __syncthreads();
  if (flags[0]) {
    __threadfence();
    for (int r = tid; r < L.wo_rows; r += kAbThreads) {
      const int row = c * L.wo_rows + r;
      float s = 0.f;
      for (int gg = 0; gg < p.G; ++gg) s += __ldcg(p.partial + (size_t)gg * E + row);
      const float v = __fadd_rn(round_bf16(s), __bfloat162float(p.x[row]));
      p.y[row] = __float2bfloat16_rn(v);
    }
    if (tid == 0) p.counters[c] = 0;   // ready for the next launch
  }
  AB_STAMP(8);
  ab_cluster_wait();       // nobody leaves while a peer may still read its shared memory
  AB_STAMP(9);
}

template <int D, int QH>
static int launch_attn_oproj(const AttnBlockParams& p, size_t smem, cudaStream_t stream) {
  static DeviceOnce configured;   // the attribute is per device
  if (!configured.done()) {
    if (cudaFuncSetAttribute(attn_oproj_kernel<D, QH>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) !=
        cudaSuccess)
      return IRON_ERR_LAUNCH;
    configured.mark();
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(p.G * kAbCluster);
  cfg.blockDim = dim3(kAbThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = kAbCluster;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1 + pdl_attr_count();
  return cudaLaunchKernelEx(&cfg, attn_oproj_kernel<D, QH>, p) == cudaSuccess ? IRON_OK : IRON_ERR_LAUNCH;
}

// The key capacity (rows of the group's cache one CTA holds at a time) a shape runs with;
// 0 when a CTA's rows of Wo do not fit one SM's shared memory.
static int attn_oproj_kcap(int E, int H, int G, int D) {
  if (G <= 0 || H % G || E % (kAbCluster * 16)) return 0;   // whole 16-row tiles of Wo per CTA
  const int QH = H / G;
  if (QH * D > kAbThreads || G > 15) return 0;          // at most 15 clusters of eight are resident at once
  const AbLayout base = ab_layout(D, QH, E, 0);
  const long long room = 227ll * 1024 - (long long)base.total - 64;
  const long long per_key = 2ll * (D + 8) * 2 + (long long)QH * 4;
  const int cap = (int)(room / per_key) / 32 * 32;
  if (cap < 32) return 0;
  return cap > 1024 ? 1024 : cap;
}

}  // namespace iron

using namespace iron;

static unsigned long long* g_ab_trace[64] = {};   // per device; a diagnostic, off by default

extern "C" void iron_decode_attn_oproj_trace(void* d_trace) {
  const int dev = current_device();
  if (dev >= 0) g_ab_trace[dev] = static_cast<unsigned long long*>(d_trace);
}

extern "C" size_t iron_decode_attn_oproj_scratch_bytes(int E, int G) {
  if (E <= 0 || G <= 0) return 0;
  return (size_t)G * E * sizeof(float) + 256;
}

extern "C" int iron_decode_attn_oproj_supported(int E, int H, int G, int D) {
  if ((D != 64 && D != 128) || G <= 0 || H % G) return 0;
  const int QH = H / G;
  if (QH != 1 && QH != 2 && QH != 4) return 0;
  return attn_oproj_kcap(E, H, G, D);
}

extern "C" int iron_decode_attn_oproj_bf16(const void* q, const void* Wo, const void* x, int position,
                                           const int* d_position, const void* k_cache, const void* v_cache,
                                           void* y, int E, int H, int G, int D, int cache_rows, int window,
                                           float scale, void* scratch, int* d_status, iron_stream_t stream) {
  if (E <= 0 || H <= 0 || G <= 0 || cache_rows <= 0 || H % G) return IRON_ERR_SHAPE;
  if (!q || !Wo || !x || !k_cache || !v_cache || !y || !scratch) return IRON_ERR_SHAPE;
  if (!d_position && (position < 0 || position >= cache_rows)) return IRON_ERR_SHAPE;
  if (!aligned16(q) || !aligned16(Wo) || !aligned16(x) || !aligned16(k_cache) || !aligned16(v_cache) ||
      !aligned16(y) || !aligned16(scratch))
    return IRON_ERR_ALIGN;
  const int kcap = iron_decode_attn_oproj_supported(E, H, G, D);
  if (!kcap) return IRON_ERR_UNSUPPORTED;
  const int QH = H / G;
  AttnBlockParams p = {};
  p.q = (const __nv_bfloat16*)q; p.wo = (const __nv_bfloat16*)Wo; p.x = (const __nv_bfloat16*)x;
  p.k_cache = (const __nv_bfloat16*)k_cache; p.v_cache = (const __nv_bfloat16*)v_cache; p.y = (__nv_bfloat16*)y;
  p.partial = reinterpret_cast<float*>(static_cast<unsigned char*>(scratch) + 256);
  p.counters = reinterpret_cast<unsigned int*>(scratch);
  p.d_position = d_position; p.position = position;
  p.E = E; p.H = H; p.G = G; p.cache_rows = cache_rows; p.window = window; p.kcap = kcap;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.status = d_status;
  p.trace = current_device() >= 0 ? g_ab_trace[current_device()] : nullptr;
  const size_t smem = ab_layout(D, QH, E, kcap).total;
  cudaStream_t s = (cudaStream_t)stream;
#define IRON_AB_CASE(DD, QQ) if (D == DD && QH == QQ) return launch_attn_oproj<DD, QQ>(p, smem, s);
  IRON_AB_CASE(64, 4) IRON_AB_CASE(64, 2) IRON_AB_CASE(64, 1)
  IRON_AB_CASE(128, 2) IRON_AB_CASE(128, 1)
#undef IRON_AB_CASE
  return IRON_ERR_UNSUPPORTED;
}
