// One decode step's attention block of a Llama-style layer in ONE kernel:
//
//     y = x + Wo . attention( RoPE(Wq . h), cache ++ RoPE(Wk . h), cache ++ Wv . h ),  h = RMSNorm(x) * w
//
// i.e. the reference's steps input_layernorm, q/k/v projections, two RoPE, two cache writes,
// MHA, o_proj and the residual add (iron/lm/blocks.py:627-648, :472-502, :723-728) -- three
// dependent launches of the separate-kernel path (fused QKV GEMV, split-K attention, o_proj
// GEMV), each of which costs a few microseconds of launch-to-launch latency while moving
// 2-13 MB.  Nothing between them needs the whole GPU to agree except the final sum, because
// the work splits by KV group: the q heads of group g need only k and v of group g, and
// their share of o_proj is the 'QH * D' columns of Wo that multiply their outputs.
//
// So a thread-block cluster owns one KV group.  Its CTAs
//   1. (before the dependency wait) start every byte they will need on its way into shared
//      memory: their rows of Wq/Wk/Wv and their rows of the group's column block of Wo by
//      bulk copies (cp.async.bulk + mbarrier), their slice of the group's cached keys and
//      values by 16-byte asynchronous copies.  None of it depends on the previous kernel;
//   2. wait for x, normalise it (two roundings, as the RMSNorm operator), compute their q/k/v
//      rows from shared memory, rotate q and k, write k and v to the cache and hand all
//      'QH + 2' head rows to every CTA of the cluster over distributed shared memory;
//   3. (cluster barrier) run the one-query attention of the group's heads over their slice
//      of the keys, merge the slices' (max, sum, output) over distributed shared memory
//      (cluster barrier) -- every CTA then holds the group's attention output;
//   4. multiply their rows of Wo's column block by it: a float32 partial of y per group,
//      written to a scratch the caller provides.
// The last cluster to finish (an arrival counter; nobody waits for anybody) adds the G
// partials in group order, rounds as the o_proj GEMV's output rounds, adds the residual and
// rounds again.  Every wait on a copy is bounded; a wait that gives up records
// IRON_ERR_TIMEOUT and the CTA walks on through the same barriers, so a lost copy costs a
// wrong vector and an error status, never a hang.
#include <cooperative_groups.h>

#include "common.cuh"
#include "gemv_items.cuh"

namespace cg = cooperative_groups;

namespace iron {

constexpr int kAbThreads = 256;
constexpr int kAbWarps = kAbThreads / 32;
constexpr unsigned long long kAbWaitNs = 2000000000ull;   // 2 s

struct AttnBlockParams {
  const __nv_bfloat16* wqkv;     // ((H + 2G) * D, E): q rows, k rows, v rows
  const __nv_bfloat16* wo;       // (E, H * D)
  const __nv_bfloat16* x;        // (E) the residual stream
  const __nv_bfloat16* norm_w;   // (E)
  const __nv_bfloat16* angles;   // (cache_rows, D) cos at even, sin at odd columns
  __nv_bfloat16* k_cache;        // (cache_rows, G, D)
  __nv_bfloat16* v_cache;
  __nv_bfloat16* y;              // (E)
  float* partial;                // (G, E) scratch
  unsigned int* counter;         // one word, zero between launches
  const int* d_position;
  int position;
  int E, H, G, cache_rows, window, kcap;
  float eps, scale_log2;
  int* status;
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

// Shared-memory plan of one CTA (bytes), for the host's size check and the kernel's carving.
struct AbLayout {
  int w_rows, wo_rows, wo_cols;
  size_t off_w, off_wo, off_k, off_v, off_x, off_qkv, off_part, off_att, off_so, off_ml, off_misc, total;
};
__host__ __device__ inline AbLayout ab_layout(int D, int QH, int E, int NC, int kcap) {
  AbLayout L;
  L.w_rows = (QH + 2) * D / NC;
  L.wo_rows = E / NC;
  L.wo_cols = QH * D;
  size_t o = 0;
  auto take = [&o](size_t bytes) { const size_t at = o; o += (bytes + 15) & ~(size_t)15; return at; };
  L.off_w = take((size_t)L.w_rows * E * 2);
  L.off_wo = take((size_t)L.wo_rows * L.wo_cols * 2);
  L.off_k = take((size_t)kcap * D * 2);
  L.off_v = take((size_t)kcap * D * 2);
  L.off_x = take((size_t)E * 2);
  L.off_qkv = take((size_t)(QH + 2) * D * 4);
  L.off_part = take((size_t)QH * (D + 2) * 4);
  L.off_att = take((size_t)QH * D * 2);
  L.off_so = take((size_t)kAbWarps * QH * D * 4);
  L.off_ml = take((size_t)kAbWarps * QH * 2 * 4);
  L.off_misc = take(128 + 32 * 4);   // two mbarriers and two flags, then the block-sum scratch
  L.total = o;
  return L;
}

template <int D, int QH>
__global__ void __launch_bounds__(kAbThreads, 1) attn_block_kernel(const AttnBlockParams p) {
  extern __shared__ __align__(128) unsigned char ab_smem[];
  cg::cluster_group cluster = cg::this_cluster();
  const int NC = (int)cluster.num_blocks();
  const int c = (int)cluster.block_rank();
  const int g = blockIdx.x / NC;                       // KV group of this cluster
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int E = p.E;
  constexpr int R = (QH + 2) * D;                      // head rows of a group: q heads, k, v
  constexpr int HALF = D / 2;
  const AbLayout L = ab_layout(D, QH, E, NC, p.kcap);
  __nv_bfloat16* wsm = reinterpret_cast<__nv_bfloat16*>(ab_smem + L.off_w);
  __nv_bfloat16* wosm = reinterpret_cast<__nv_bfloat16*>(ab_smem + L.off_wo);
  __nv_bfloat16* ksm = reinterpret_cast<__nv_bfloat16*>(ab_smem + L.off_k);
  __nv_bfloat16* vsm = reinterpret_cast<__nv_bfloat16*>(ab_smem + L.off_v);
  uint4* xs = reinterpret_cast<uint4*>(ab_smem + L.off_x);
  float* qkv = reinterpret_cast<float*>(ab_smem + L.off_qkv);            // [R] after RoPE, bf16 values
  float* part = reinterpret_cast<float*>(ab_smem + L.off_part);          // [QH][D + 2]
  __nv_bfloat16* att = reinterpret_cast<__nv_bfloat16*>(ab_smem + L.off_att);   // [QH * D]
  float* sm_o = reinterpret_cast<float*>(ab_smem + L.off_so);            // [warps][QH][D]
  float* sm_ml = reinterpret_cast<float*>(ab_smem + L.off_ml);           // [warps][QH][2]
  uint64_t* bars = reinterpret_cast<uint64_t*>(ab_smem + L.off_misc);    // [0] q/k/v rows, [1] Wo rows
  int* flags = reinterpret_cast<int*>(bars + 2);                         // [0] last cluster, [1] a wait gave up
  float* red = reinterpret_cast<float*>(ab_smem + L.off_misc + 128);

  if (tid == 0) {
    ab_mbar_init(bars);
    ab_mbar_init(bars + 1);
    flags[0] = 0; flags[1] = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  pdl_launch();

  // ---- 1. everything this CTA will read, on its way before the dependency resolves ----
  // unit u of the group: head hh = u / HALF (q heads, then k, then v), pair (i, i + HALF)
  const int upc = R / 2 / NC;                          // units of this CTA
  auto weight_row = [&](int hh, int i) -> size_t {
    const int head = hh < QH ? g * QH + hh : (hh == QH ? p.H + g : p.H + p.G + g);
    return (size_t)head * D + i;
  };
  uint64_t policy;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
  if (warp == 0) {
    if (lane == 0) ab_expect_tx(bars, (uint32_t)(2 * upc) * (uint32_t)E * 2u);
    __syncwarp();
    for (int s = lane; s < 2 * upc; s += 32) {
      const int u = c * upc + (s >> 1);
      const int hh = u / HALF, i = u - hh * HALF + (s & 1) * HALF;
      ab_bulk_load(wsm + (size_t)s * E, p.wqkv + weight_row(hh, i) * E, (uint32_t)E * 2u, bars, policy);
    }
  } else if (warp == 1) {
    if (lane == 0) ab_expect_tx(bars + 1, (uint32_t)L.wo_rows * (uint32_t)L.wo_cols * 2u);
    __syncwarp();
    const size_t pitch = (size_t)p.H * D;
    for (int r = lane; r < L.wo_rows; r += 32)
      ab_bulk_load(wosm + (size_t)r * L.wo_cols, p.wo + (size_t)(c * L.wo_rows + r) * pitch + (size_t)g * L.wo_cols,
                   (uint32_t)L.wo_cols * 2u, bars + 1, policy);
  }
  // The position was written by the draw of the previous step, kernels ago; it is read again
  // after the wait, and the keys are fetched again if it was not yet there.
  auto key_range = [&](int pos, int& lo_all, int& kb, int& ke) {
    const int kv_valid = pos + 1;
    lo_all = (p.window >= 0) ? max(0, kv_valid - 1 - p.window) : 0;
    const int per = (kv_valid - lo_all + NC - 1) / NC;
    kb = lo_all + c * per;
    ke = min(kv_valid, kb + per);
  };
  auto fetch_keys = [&](int k0, int k1, int pos) {     // cache rows [k0, k1) but the newest
    const int n = k1 - k0;
    constexpr int CH = D / 8;
    for (int idx = tid; idx < n * CH; idx += kAbThreads) {
      const int j = idx / CH, ch = idx - j * CH;
      if (k0 + j == pos) continue;
      const size_t src = ((size_t)(k0 + j) * p.G + g) * D + ch * 8;
      ab_cp16(ksm + (size_t)j * D + ch * 8, p.k_cache + src);
      ab_cp16(vsm + (size_t)j * D + ch * 8, p.v_cache + src);
    }
  };
  const int pos_early = min(max(p.d_position ? *p.d_position : p.position, 0), p.cache_rows - 1);
  int lo_all, kb, ke;
  key_range(pos_early, lo_all, kb, ke);
  fetch_keys(kb, min(ke, kb + p.kcap), pos_early);

  pdl_wait();

  // ---- 2. h = RMSNorm(x) * w, this CTA's q/k/v rows, RoPE, the cache rows, the hand-over ----
  const int pos = min(max(p.d_position ? *p.d_position : p.position, 0), p.cache_rows - 1);
  const int nch = E >> 3;
  {
    const uint4* xg = reinterpret_cast<const uint4*>(p.x);
    float ss = 0.f;
    for (int i = tid; i < nch; i += kAbThreads) {
      const uint4 v = ld_cached(xg + i);
      xs[i] = v;
      float f[8];
      unpack8(v, f);
#pragma unroll
      for (int j = 0; j < 8; ++j) ss = fmaf(f[j], f[j], ss);
    }
    const float tot = block_sum(ss, red);
    const float inv = 1.0f / sqrtf(tot / (float)E + p.eps);
    const uint4* wg = reinterpret_cast<const uint4*>(p.norm_w);
    for (int i = tid; i < nch; i += kAbThreads) {
      float f[8], w[8];
      unpack8(xs[i], f);
      unpack8(ld_cached(wg + i), w);
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] = round_bf16(f[j] * inv) * w[j];
      xs[i] = pack8(f);
    }
    __syncthreads();
  }
  bool ok = ab_wait(bars);
  for (int ul = warp; ul < upc; ul += kAbWarps) {
    const uint4* wa = reinterpret_cast<const uint4*>(wsm + (size_t)(2 * ul) * E);
    const uint4* wb = reinterpret_cast<const uint4*>(wsm + (size_t)(2 * ul + 1) * E);
    float a0 = 0.f, a1 = 0.f, b0 = 0.f, b1 = 0.f;
    for (int i = lane; i < nch; i += 64) {
      const uint4 x0 = xs[i];
      a0 = dot8(wa[i], x0, a0);
      b0 = dot8(wb[i], x0, b0);
      if (i + 32 < nch) {
        const uint4 x1 = xs[i + 32];
        a1 = dot8(wa[i + 32], x1, a1);
        b1 = dot8(wb[i + 32], x1, b1);
      }
    }
    const float acc0 = warp_sum(a0 + a1), acc1 = warp_sum(b0 + b1);
    const int u = c * upc + ul;
    const int hh = u / HALF, i = u - hh * HALF;
    float x1 = round_bf16(acc0), x2 = round_bf16(acc1);
    if (hh <= QH) {   // q heads and k rotate
      const __nv_bfloat16* ang = p.angles + (size_t)pos * D;
      const float cs = __bfloat162float(ang[2 * i]), sn = __bfloat162float(ang[2 * i + 1]);
      const float y1 = __fsub_rn(__fmul_rn(x1, cs), __fmul_rn(x2, sn));
      const float y2 = __fadd_rn(__fmul_rn(x2, cs), __fmul_rn(x1, sn));
      x1 = y1; x2 = y2;
    }
    x1 = round_bf16(x1); x2 = round_bf16(x2);
    if (lane == 0 && hh >= QH) {
      __nv_bfloat16* dst = (hh == QH ? p.k_cache : p.v_cache) + ((size_t)pos * p.G + g) * D;
      dst[i] = __float2bfloat16_rn(x1);
      dst[i + HALF] = __float2bfloat16_rn(x2);
    }
    if (lane < NC) {   // every CTA of the cluster gets the pair
      float* remote = cluster.map_shared_rank(qkv, lane);
      remote[hh * D + i] = x1;
      remote[hh * D + i + HALF] = x2;
    }
  }
  cluster.sync();

  // ---- 3. attention of the group's heads over this CTA's keys ----
  key_range(pos, lo_all, kb, ke);
  constexpr int LPK = D / 8, KPW = 32 / LPK, TS = KPW * kAbWarps;
  const int dsel = lane % LPK, kslot = warp * KPW + lane / LPK;
  float q[QH][8], o[QH][8], m[QH], l[QH];
#pragma unroll
  for (int h = 0; h < QH; ++h) {
    m[h] = -INFINITY; l[h] = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) { o[h][j] = 0.f; q[h][j] = qkv[h * D + dsel * 8 + j] * p.scale_log2; }
  }
  bool first = (pos == pos_early);
  for (int cs = kb; cs < ke; cs += p.kcap) {
    const int ce = min(ke, cs + p.kcap);
    if (!first) {   // a later chunk (or keys fetched for a stale position): the buffers are reused
      ab_cp_wait_all();
      __syncthreads();
      fetch_keys(cs, ce, pos);
    }
    first = false;
    ab_cp_wait_all();
    if (pos >= cs && pos < ce)    // the newest row comes from this step, not from the cache
      for (int e = tid; e < 2 * D; e += kAbThreads) {
        __nv_bfloat16* dst = (e < D ? ksm : vsm) + (size_t)(pos - cs) * D + (e < D ? e : e - D);
        *dst = __float2bfloat16_rn(qkv[(QH + (e < D ? 0 : 1)) * D + (e < D ? e : e - D)]);
      }
    __syncthreads();
    const int n = ce - cs;
    for (int j0 = 0; j0 < n; j0 += TS) {
      const int j = j0 + kslot;
      const bool live = j < n;
      const int jj = live ? j : n - 1;
      float kf[8], vf[8];
      unpack8(*reinterpret_cast<const uint4*>(ksm + (size_t)jj * D + dsel * 8), kf);
      unpack8(*reinterpret_cast<const uint4*>(vsm + (size_t)jj * D + dsel * 8), vf);
#pragma unroll
      for (int h = 0; h < QH; ++h) {
        float a = 0.f;
#pragma unroll
        for (int e = 0; e < 8; ++e) a = fmaf(q[h][e], kf[e], a);
#pragma unroll
        for (int off = 1; off < LPK; off <<= 1) a += __shfl_xor_sync(0xffffffffu, a, off);
        if (!live) continue;
        const float mn = fmaxf(m[h], a);
        const float corr = exp2f(m[h] - mn), pr = exp2f(a - mn);
        l[h] = fmaf(l[h], corr, pr);
#pragma unroll
        for (int e = 0; e < 8; ++e) o[h][e] = fmaf(pr, vf[e], o[h][e] * corr);
        m[h] = mn;
      }
    }
  }
  // merge the lane groups of a warp, then the warps, into this CTA's partial
#pragma unroll
  for (int off = LPK; off < 32; off <<= 1) {
#pragma unroll
    for (int h = 0; h < QH; ++h) {
      const float mo = __shfl_xor_sync(0xffffffffu, m[h], off);
      const float lo2 = __shfl_xor_sync(0xffffffffu, l[h], off);
      const float mn = fmaxf(m[h], mo);
      const float ca = (m[h] == -INFINITY) ? 0.f : exp2f(m[h] - mn);
      const float cb = (mo == -INFINITY) ? 0.f : exp2f(mo - mn);
      l[h] = l[h] * ca + lo2 * cb;
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float oo = __shfl_xor_sync(0xffffffffu, o[h][e], off);
        o[h][e] = o[h][e] * ca + oo * cb;
      }
      m[h] = mn;
    }
  }
  if (lane < LPK) {
#pragma unroll
    for (int h = 0; h < QH; ++h) {
#pragma unroll
      for (int e = 0; e < 8; ++e) sm_o[(warp * QH + h) * D + dsel * 8 + e] = o[h][e];
      if (lane == 0) { sm_ml[(warp * QH + h) * 2] = m[h]; sm_ml[(warp * QH + h) * 2 + 1] = l[h]; }
    }
  }
  __syncthreads();
  for (int e = tid; e < QH * D; e += kAbThreads) {
    const int h = e / D, d = e - h * D;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < kAbWarps; ++w) M = fmaxf(M, sm_ml[(w * QH + h) * 2]);
    float Ls = 0.f, acc = 0.f;
#pragma unroll
    for (int w = 0; w < kAbWarps; ++w) {
      const float mw = sm_ml[(w * QH + h) * 2];
      const float cf = (mw == -INFINITY) ? 0.f : exp2f(mw - M);
      Ls = fmaf(sm_ml[(w * QH + h) * 2 + 1], cf, Ls);
      acc = fmaf(sm_o[(w * QH + h) * D + d], cf, acc);
    }
    part[h * (D + 2) + d] = acc;
    if (d == 0) { part[h * (D + 2) + D] = M; part[h * (D + 2) + D + 1] = Ls; }
  }
  cluster.sync();
  // every CTA folds the cluster's partials: it needs the whole output for its rows of Wo
  for (int e = tid; e < QH * D; e += kAbThreads) {
    const int h = e / D, d = e - h * D;
    float M = -INFINITY;
    for (int r = 0; r < NC; ++r) M = fmaxf(M, cluster.map_shared_rank(part, r)[h * (D + 2) + D]);
    float Ls = 0.f, acc = 0.f;
    for (int r = 0; r < NC; ++r) {
      const float* remote = cluster.map_shared_rank(part, r);
      const float ms = remote[h * (D + 2) + D];
      const float cf = (ms == -INFINITY) ? 0.f : exp2f(ms - M);
      Ls = fmaf(remote[h * (D + 2) + D + 1], cf, Ls);
      acc = fmaf(remote[h * (D + 2) + d], cf, acc);
    }
    att[e] = __float2bfloat16_rn(Ls > 0.f ? acc / Ls : 0.f);
  }
  __syncthreads();

  // ---- 4. this CTA's rows of Wo's column block times the group's output ----
  ok = ab_wait(bars + 1) && ok;
  {
    const int c16 = L.wo_cols >> 3;
    const uint4* av = reinterpret_cast<const uint4*>(att);
    for (int r = warp; r < L.wo_rows; r += kAbWarps) {
      const uint4* wr = reinterpret_cast<const uint4*>(wosm + (size_t)r * L.wo_cols);
      float a = 0.f;
      for (int i = lane; i < c16; i += 32) a = dot8(wr[i], av[i], a);
      a = warp_sum(a);
      if (lane == 0) p.partial[(size_t)g * E + c * L.wo_rows + r] = a;
    }
  }
  if (!ok && tid == 0 && p.status) *reinterpret_cast<volatile int*>(p.status) = IRON_ERR_TIMEOUT;
  __threadfence();
  cluster.sync();   // the cluster's partial is complete (and nobody reads a peer's shared memory any more)
  if (c == 0 && tid == 0) {
    const unsigned int arrived = atomicAdd(p.counter, 1u);
    const int last = arrived == (unsigned int)p.G - 1;
    for (int r = 0; r < NC; ++r) cluster.map_shared_rank(flags, r)[0] = last;
  }
  cluster.sync();
  if (flags[0]) {   // the last cluster adds the groups' partials in order, rounds, adds the residual
    __threadfence();
    for (int r = tid; r < L.wo_rows; r += kAbThreads) {
      const int row = c * L.wo_rows + r;
      float s = 0.f;
      for (int gg = 0; gg < p.G; ++gg) s += __ldcg(p.partial + (size_t)gg * E + row);
      const float v = __fadd_rn(round_bf16(s), __bfloat162float(p.x[row]));
      p.y[row] = __float2bfloat16_rn(v);
    }
    if (c == 0 && tid == 0) *p.counter = 0;   // ready for the next launch
  }
}

template <int D, int QH>
static int launch_attn_block(const AttnBlockParams& p, int NC, size_t smem, cudaStream_t stream) {
  static DeviceOnce configured;
  if (!configured.done()) {
    if (cudaFuncSetAttribute(attn_block_kernel<D, QH>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) !=
            cudaSuccess ||
        cudaFuncSetAttribute(attn_block_kernel<D, QH>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) !=
            cudaSuccess)
      return IRON_ERR_LAUNCH;
    configured.mark();
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(p.G * NC);
  cfg.blockDim = dim3(kAbThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = NC;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1 + pdl_attr_count();
  return cudaLaunchKernelEx(&cfg, attn_block_kernel<D, QH>, p) == cudaSuccess ? IRON_OK : IRON_ERR_LAUNCH;
}

// The cluster size and key capacity a shape runs with; 0 when its rows do not fit one SM.
static int attn_block_plan(int E, int H, int G, int D, int* kcap) {
  if (G <= 0 || H % G) return 0;
  const int QH = H / G;
  for (int NC = 16; NC >= 8; NC >>= 1) {
    if (((QH + 2) * D / 2) % NC || E % NC || (E & 7)) continue;
    const AbLayout base = ab_layout(D, QH, E, NC, 0);
    const long long room = 227ll * 1024 - (long long)base.total;
    const int cap = (int)(room / (2ll * D * 2)) / 32 * 32;
    if (cap < 32) continue;
    *kcap = cap > 1024 ? 1024 : cap;
    return NC;
  }
  return 0;
}

}  // namespace iron

using namespace iron;

extern "C" size_t iron_decode_attn_block_scratch_bytes(int E, int G) {
  if (E <= 0 || G <= 0) return 0;
  return (size_t)G * E * sizeof(float) + 256;
}

extern "C" int iron_decode_attn_block_supported(int E, int H, int G, int D) {
  int kcap = 0;
  if ((D != 64 && D != 128) || G <= 0 || H % G) return 0;
  const int QH = H / G;
  if (!((D == 64 && (QH == 4 || QH == 2 || QH == 1)) || (D == 128 && (QH == 4 || QH == 2 || QH == 1)))) return 0;
  return attn_block_plan(E, H, G, D, &kcap);
}

extern "C" int iron_decode_attn_block_bf16(const void* Wqkv, const void* Wo, const void* x, const void* norm_weight,
                                           float eps, const void* angles, int position, const int* d_position,
                                           void* k_cache, void* v_cache, void* y, int E, int H, int G, int D,
                                           int cache_rows, int window, float scale, void* scratch,
                                           int* d_status, iron_stream_t stream) {
  if (E <= 0 || H <= 0 || G <= 0 || cache_rows <= 0 || H % G) return IRON_ERR_SHAPE;
  if (!Wqkv || !Wo || !x || !norm_weight || !angles || !k_cache || !v_cache || !y || !scratch) return IRON_ERR_SHAPE;
  if (!d_position && (position < 0 || position >= cache_rows)) return IRON_ERR_SHAPE;
  if (!aligned16(Wqkv) || !aligned16(Wo) || !aligned16(x) || !aligned16(norm_weight) || !aligned16(k_cache) ||
      !aligned16(v_cache) || !aligned16(y) || !aligned16(scratch))
    return IRON_ERR_ALIGN;
  int kcap = 0;
  const int NC = iron_decode_attn_block_supported(E, H, G, D) ? attn_block_plan(E, H, G, D, &kcap) : 0;
  if (!NC) return IRON_ERR_UNSUPPORTED;
  const int QH = H / G;
  AttnBlockParams p = {};
  p.wqkv = (const __nv_bfloat16*)Wqkv; p.wo = (const __nv_bfloat16*)Wo; p.x = (const __nv_bfloat16*)x;
  p.norm_w = (const __nv_bfloat16*)norm_weight; p.angles = (const __nv_bfloat16*)angles;
  p.k_cache = (__nv_bfloat16*)k_cache; p.v_cache = (__nv_bfloat16*)v_cache; p.y = (__nv_bfloat16*)y;
  p.partial = reinterpret_cast<float*>(static_cast<unsigned char*>(scratch) + 256);
  p.counter = reinterpret_cast<unsigned int*>(scratch);
  p.d_position = d_position; p.position = position;
  p.E = E; p.H = H; p.G = G; p.cache_rows = cache_rows; p.window = window; p.kcap = kcap;
  p.eps = eps; p.scale_log2 = scale * 1.4426950408889634f;
  p.status = d_status;
  const size_t smem = ab_layout(D, QH, E, NC, kcap).total;
  cudaStream_t s = (cudaStream_t)stream;
#define IRON_AB_CASE(DD, QQ) if (D == DD && QH == QQ) return launch_attn_block<DD, QQ>(p, NC, smem, s);
  IRON_AB_CASE(64, 4) IRON_AB_CASE(64, 2) IRON_AB_CASE(64, 1)
  IRON_AB_CASE(128, 4) IRON_AB_CASE(128, 2) IRON_AB_CASE(128, 1)
#undef IRON_AB_CASE
  return IRON_ERR_UNSUPPORTED;
}
