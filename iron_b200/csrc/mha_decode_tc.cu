// One-query attention for a *batch* of sequences on the warp tensor cores.
//
// When the batch alone fills the machine (batch x KV heads >= two CTAs per SM) the SIMT
// decode kernel is bound by instruction issue: every key costs a dot product and an
// accumulation per query head.  Here the query heads that share a KV head are the rows of
// one 16-row MMA tile, so K and V are read once for the whole group and the arithmetic runs
// as mma.sync m16n8k16:
//   one CTA = one (sequence, KV head); 4 warps; keys stream through shared memory in
//   64-row tiles (cp.async, double buffered, XOR-swizzled 16-byte chunks); within a tile
//   each warp takes 16 keys: S = Q K^T (2 key tiles x D/16 steps), online softmax in the
//   exp2 domain, O += P V (D/8 column tiles); the four warps' (max, sum, O) are merged
//   through shared memory at the end.
// Rows of the tile beyond the group are zero queries whose results are dropped.
//
// A batch that does not fill the machine that way (8 sequences x 8 KV heads = 64 CTAs on 148 SMs) is
// split along the keys as well: a thread-block cluster of 2, 4 or 8 CTAs shares one (sequence, KV head),
// each takes a contiguous run of key tiles, leaves its (O, max, sum) in its shared memory, and after one
// cluster barrier every CTA merges its slice of the outputs over distributed shared memory.
#include <cooperative_groups.h>

#include "common.cuh"

namespace iron {

struct DecodeTcParams {
  const __nv_bfloat16* Q;   // (B, H, D)
  const __nv_bfloat16* K;
  const __nv_bfloat16* V;
  __nv_bfloat16* O;         // (B, H, D)
  long long kv_batch_stride, kv_seq_stride, kv_head_stride;  // elements
  int H, G, group;
  int kv_valid;
  const int* d_kv_valid;
  int d_kv_valid_stride;
  int kv_valid_add;
  int kv_max;
  int window;               // < 0: none
  float scale_log2;
  int nsplit;               // CTAs (a cluster along z) that share the keys of one (sequence, KV head)
  int tiles_cap;            // resident form: key tiles one CTA holds
  int stable_prefix;        // resident form: only the newest cache row was written by the kernel just before
};

constexpr int kDtThreads = 128;
constexpr int kDtKeys = 64;   // keys per shared-memory tile

__device__ __forceinline__ void dt_cp_async16(uint32_t dst, const void* src, bool pred) {
  const int bytes = pred ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void dt_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void dt_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void dt_ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void dt_ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2,
                                                     uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void dt_mma(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float dt_ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t dt_pack(float a, float b) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&v);
}
// Byte offset of 16-byte chunk `chunk` of row `row` in a tile whose rows are D bf16 wide.
template <int D>
__device__ __forceinline__ uint32_t dt_swz(int row, int chunk) {
  return (uint32_t)(row * (D * 2) + ((((chunk & 7) ^ (row & 7)) | (chunk & ~7)) << 4));
}

// One 64-key tile (K at kt_base, V at vt_base in shared memory, first key tile_key0): this warp's 16
// keys go through S = Q K^T, the online softmax and O += P V.
template <int D>
__device__ __forceinline__ void dt_tile(uint32_t kt_base, uint32_t vt_base, int tile_key0, int kv_valid, int lo,
                                        float scale_log2, int warp, int lane, const uint32_t (&qf)[D / 16][4],
                                        float (&o)[D / 8][4], float (&m_run)[2], float (&l_run)[2]) {
  const int t = lane & 3;
  // ---- S = Q K^T for this warp's 16 keys of the tile ----
  float s[2][4];
#pragma unroll
  for (int nt = 0; nt < 2; ++nt) { s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f; }
#pragma unroll
  for (int kt = 0; kt < D / 16; ++kt) {
    uint32_t b0, b1, b2, b3;
    const int row = warp * 16 + (lane & 7) + (lane >> 4) * 8;
    dt_ldmatrix_x4(kt_base + dt_swz<D>(row, kt * 2 + ((lane >> 3) & 1)), b0, b1, b2, b3);
    dt_mma(s[0], qf[kt], b0, b1);
    dt_mma(s[1], qf[kt], b2, b3);
  }
  // ---- mask, online softmax (rows g and g + 8 of the tile) ----
  const int key0 = tile_key0 + warp * 16;
  float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
  for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int key = key0 + nt * 8 + 2 * t + (e & 1);
      float v = s[nt][e] * scale_log2;
      if (key >= kv_valid || key < lo) v = -INFINITY;
      s[nt][e] = v;
      mx[e >> 1] = fmaxf(mx[e >> 1], v);
    }
  }
  float corr[2], msafe[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
    mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
    const float mn = fmaxf(m_run[r], mx[r]);
    msafe[r] = (mn == -INFINITY) ? 0.f : mn;
    corr[r] = dt_ex2(m_run[r] - msafe[r]);
    m_run[r] = mn;
    l_run[r] *= corr[r];
  }
  uint32_t pf[4];
  {
    const float p00 = dt_ex2(s[0][0] - msafe[0]), p01 = dt_ex2(s[0][1] - msafe[0]);
    const float p02 = dt_ex2(s[0][2] - msafe[1]), p03 = dt_ex2(s[0][3] - msafe[1]);
    const float p10 = dt_ex2(s[1][0] - msafe[0]), p11 = dt_ex2(s[1][1] - msafe[0]);
    const float p12 = dt_ex2(s[1][2] - msafe[1]), p13 = dt_ex2(s[1][3] - msafe[1]);
    l_run[0] += (p00 + p01) + (p10 + p11);
    l_run[1] += (p02 + p03) + (p12 + p13);
    pf[0] = dt_pack(p00, p01); pf[1] = dt_pack(p02, p03);
    pf[2] = dt_pack(p10, p11); pf[3] = dt_pack(p12, p13);
  }
#pragma unroll
  for (int dt = 0; dt < D / 8; ++dt) {
    o[dt][0] *= corr[0]; o[dt][1] *= corr[0];
    o[dt][2] *= corr[1]; o[dt][3] *= corr[1];
  }
  // ---- O += P V over this warp's 16 keys ----
#pragma unroll
  for (int dp = 0; dp < D / 16; ++dp) {
    uint32_t b0, b1, b2, b3;
    const int row = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
    dt_ldmatrix_x4_trans(vt_base + dt_swz<D>(row, dp * 2 + (lane >> 4)), b0, b1, b2, b3);
    dt_mma(o[2 * dp], pf, b0, b1);
    dt_mma(o[2 * dp + 1], pf, b2, b3);
  }
}

// The query heads of a KV head as MMA fragments, from the 16-row tile at sQ.
template <int D>
__device__ __forceinline__ void dt_load_q(uint32_t sQ, int lane, uint32_t (&qf)[D / 16][4]) {
#pragma unroll
  for (int kt = 0; kt < D / 16; ++kt) {
    const int row = (lane & 7) + ((lane >> 3) & 1) * 8;
    dt_ldmatrix_x4(sQ + dt_swz<D>(row, kt * 2 + (lane >> 4)), qf[kt][0], qf[kt][1], qf[kt][2], qf[kt][3]);
  }
}

// Every warp's (O, max, sum) for rows g and g + 8 into `part` ([warp][16 rows][D + 2] floats).
template <int D>
__device__ __forceinline__ void dt_park(float* part, int warp, int lane, const float (&o)[D / 8][4],
                                        const float (&m_run)[2], const float (&l_run)[2]) {
  constexpr int kRow = D + 2;
  const int g = lane >> 2, t = lane & 3;
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    float l = l_run[r];
    l += __shfl_xor_sync(0xffffffffu, l, 1);
    l += __shfl_xor_sync(0xffffffffu, l, 2);
    const int row = g + r * 8;
    float* dst = part + ((size_t)warp * 16 + row) * kRow;
#pragma unroll
    for (int dt = 0; dt < D / 8; ++dt) {
      dst[dt * 8 + 2 * t] = o[dt][2 * r];
      dst[dt * 8 + 2 * t + 1] = o[dt][2 * r + 1];
    }
    if (t == 0) { dst[D] = m_run[r]; dst[D + 1] = l; }
  }
}

// The four warps' partials of `part` folded into one (O, max, sum) per query head at `mine`
// ([group][D + 2]: D outputs, the maximum, the sum).
template <int D, int NW = 4>
__device__ __forceinline__ void dt_fold_warps(const float* part, float* mine, int group, int tid, int threads = kDtThreads) {
  constexpr int kRow = D + 2;
  for (int idx = tid; idx < group * kRow; idx += threads) {
    const int row = idx / kRow, d = idx - row * kRow;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < NW; ++w) M = fmaxf(M, part[((size_t)w * 16 + row) * kRow + D]);
    float v = 0.f;
    if (d == D) v = M;
    else {
      const int col = d < D ? d : D + 1;      // an output, or the sum
#pragma unroll
      for (int w = 0; w < NW; ++w) {
        const float* src = part + ((size_t)w * 16 + row) * kRow;
        const float c = (src[D] == -INFINITY) ? 0.f : dt_ex2(src[D] - M);
        v = fmaf(src[col], c, v);
      }
    }
    mine[idx] = v;
  }
}

template <int D>
__global__ void __launch_bounds__(kDtThreads) mha_decode_tc_kernel(const DecodeTcParams p) {
  extern __shared__ __align__(128) uint8_t dt_smem[];
  constexpr int kTile = kDtKeys * D * 2;
  constexpr int kChunks = D / 8;
  const uint32_t sQ = smem_u32(dt_smem);            // 16 rows x D
  const uint32_t sK = sQ + 16 * D * 2, sV = sK + 2 * kTile;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int kvh = blockIdx.x, b = blockIdx.y;

  pdl_wait();
  pdl_launch();

  int kv_valid = p.kv_valid;
  if (p.d_kv_valid) kv_valid = p.d_kv_valid[b * p.d_kv_valid_stride] + p.kv_valid_add;
  kv_valid = max(0, min(kv_valid, p.kv_max));
  const int lo = (p.window >= 0) ? max(0, kv_valid - 1 - p.window) : 0;
  int j_lo = lo / kDtKeys, j_hi = (kv_valid + kDtKeys - 1) / kDtKeys;
  if (p.nsplit > 1) {   // this CTA's run of key tiles
    const int per = (j_hi - j_lo + p.nsplit - 1) / p.nsplit;
    j_lo = min(j_hi, j_lo + (int)blockIdx.z * per);
    j_hi = min(j_hi, j_lo + per);
  }

  const __nv_bfloat16* Qb = p.Q + ((size_t)b * p.H + (size_t)kvh * p.group) * D;
  const __nv_bfloat16* Kb = p.K + (size_t)b * p.kv_batch_stride + (size_t)kvh * p.kv_head_stride;
  const __nv_bfloat16* Vb = p.V + (size_t)b * p.kv_batch_stride + (size_t)kvh * p.kv_head_stride;

  auto load_kv = [&](uint32_t tile, const __nv_bfloat16* base, int row0) {
#pragma unroll
    for (int i = 0; i < (kDtKeys * kChunks) / kDtThreads; ++i) {
      const int idx = tid + i * kDtThreads;
      const int r = idx / kChunks, c = idx % kChunks;
      const bool live = row0 + r < kv_valid;
      dt_cp_async16(tile + dt_swz<D>(r, c), base + (size_t)(live ? row0 + r : 0) * p.kv_seq_stride + c * 8, live);
    }
  };
  // the query heads of this KV head are rows 0 .. group-1 of the tile; the rest are zeros
  for (int idx = tid; idx < 16 * kChunks; idx += kDtThreads) {
    const int r = idx / kChunks, c = idx % kChunks;
    const bool live = r < p.group;
    dt_cp_async16(sQ + dt_swz<D>(r, c), Qb + (size_t)(live ? r : 0) * D + c * 8, live);
  }
  if (j_lo < j_hi) {
    load_kv(sK, Kb, j_lo * kDtKeys);
    load_kv(sV, Vb, j_lo * kDtKeys);
  }
  dt_commit();

  uint32_t qf[D / 16][4];
  float o[D / 8][4];
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
#pragma unroll
  for (int i = 0; i < D / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }

  for (int j = j_lo; j < j_hi; ++j) {
    const int buf = (j - j_lo) & 1;
    if (j + 1 < j_hi) {
      load_kv(sK + (buf ^ 1) * kTile, Kb, (j + 1) * kDtKeys);
      load_kv(sV + (buf ^ 1) * kTile, Vb, (j + 1) * kDtKeys);
    }
    dt_commit();
    dt_wait<1>();
    __syncthreads();
    if (j == j_lo) dt_load_q<D>(sQ, lane, qf);
    dt_tile<D>(sK + buf * kTile, sV + buf * kTile, j * kDtKeys, kv_valid, lo, p.scale_log2, warp, lane, qf, o, m_run, l_run);
    __syncthreads();  // the other buffer is overwritten by the next iteration's prefetch
  }
  dt_wait<0>();
  __syncthreads();

  // ---- merge the four warps (each saw a quarter of the keys) ----
  // per warp: 16 rows x (D outputs, max, sum) in f32, over the tiles' shared memory
  float* part = reinterpret_cast<float*>(dt_smem);
  constexpr int kRow = D + 2;
  dt_park<D>(part, warp, lane, o, m_run, l_run);
  __syncthreads();
  if (p.nsplit == 1) {
    for (int idx = tid; idx < p.group * D; idx += kDtThreads) {
      const int row = idx / D, d = idx - row * D;
      float M = -INFINITY;
#pragma unroll
      for (int w = 0; w < 4; ++w) M = fmaxf(M, part[((size_t)w * 16 + row) * kRow + D]);
      float acc = 0.f, L = 0.f;
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        const float* src = part + ((size_t)w * 16 + row) * kRow;
        const float c = (src[D] == -INFINITY) ? 0.f : dt_ex2(src[D] - M);
        acc = fmaf(src[d], c, acc);
        L = fmaf(src[D + 1], c, L);
      }
      p.O[((size_t)b * p.H + (size_t)kvh * p.group + row) * D + d] = __float2bfloat16_rn(L > 0.f ? acc / L : 0.f);
    }
    return;
  }
  // ---- keys split over the cluster: this CTA's (O, max, sum) per query head, behind the warps' partials ----
  float* mine = part + 4 * 16 * kRow;
  dt_fold_warps<D>(part, mine, p.group, tid);
  namespace cg = cooperative_groups;
  cg::cluster_group cluster = cg::this_cluster();
  cluster.sync();
  {
    const int total = p.group * D, per = (total + p.nsplit - 1) / p.nsplit;
    const int begin = (int)blockIdx.z * per, end = min(total, begin + per);
    const float* theirs[8];
#pragma unroll
    for (int r = 0; r < 8; ++r) theirs[r] = r < p.nsplit ? cluster.map_shared_rank(mine, r) : mine;
    for (int idx = begin + tid; idx < end; idx += kDtThreads) {
      const int row = idx / D, d = idx - row * D;
      float mr[8], ar[8], lr[8];
#pragma unroll
      for (int r = 0; r < 8; ++r)
        if (r < p.nsplit) {
          const float* src = theirs[r] + (size_t)row * kRow;
          mr[r] = src[D]; ar[r] = src[d]; lr[r] = src[D + 1];
        }
      float M = -INFINITY;
#pragma unroll
      for (int r = 0; r < 8; ++r)
        if (r < p.nsplit) M = fmaxf(M, mr[r]);
      float acc = 0.f, L = 0.f;
#pragma unroll
      for (int r = 0; r < 8; ++r)
        if (r < p.nsplit) {
          const float c = (mr[r] == -INFINITY) ? 0.f : dt_ex2(mr[r] - M);
          acc = fmaf(ar[r], c, acc);
          L = fmaf(lr[r], c, L);
        }
      p.O[((size_t)b * p.H + (size_t)kvh * p.group + row) * D + d] = __float2bfloat16_rn(L > 0.f ? acc / L : 0.f);
    }
  }
  cluster.sync();   // nobody leaves while a peer still reads its partial
}

// ---------------------------------------------------------------------------------------------
// The resident form, for a few sequences (fewer than 16 (sequence, KV head) pairs): latency, not
// bandwidth, is what such a launch costs, so the keys are split over as many CTAs as there are SMs
// (18 per pair for one sequence of 8 KV heads) and a CTA asks for ALL of its keys and values at
// once -- they fit its shared memory -- instead of streaming them tile after tile.  When the caller
// promises that only the newest cache row was written by the kernel just before (a decode step),
// everything else is asked for ahead of the programmatic-dependency wait, i.e. while the q/k/v
// projection still runs; after the wait come q and the newest row.  Too many CTAs for a cluster:
// every CTA leaves its (O, max, sum) in a scratch and the last to arrive for a pair (one counter per
// pair; nobody waits for anybody) folds them.  The scratch is file scope (1.2 MB per GPU, held until
// exit): launches of this form that overlap on one GPU would race -- launches of one stream do not.
constexpr int kDtResCtas = 160;                    // CTAs of a launch at most (one per SM)
constexpr int kDtResPairs = 16;
__device__ float g_dt_partial[kDtResCtas * 16 * (128 + 2)];
__device__ unsigned int g_dt_arrived[kDtResPairs];

constexpr int kDtResThreads = 256;   // two groups of four warps: a group takes every other tile

template <int D>
__global__ void __launch_bounds__(kDtResThreads) mha_decode_resident_kernel(const DecodeTcParams p) {
  extern __shared__ __align__(128) uint8_t dt_smem[];
  __shared__ int s_last;
  constexpr int kTile = kDtKeys * D * 2;
  constexpr int kChunks = D / 8;
  constexpr int kRow = D + 2;
  const uint32_t sQ = smem_u32(dt_smem);            // 16 rows x D
  const uint32_t sK = sQ + 16 * D * 2, sV = sK + p.tiles_cap * kTile;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int kvh = blockIdx.x, b = blockIdx.y, split = blockIdx.z;
  pdl_launch();
  if (!p.stable_prefix) pdl_wait();

  // the key count was written by an earlier launch (or is an immediate)
  int kv_valid = p.kv_valid;
  if (p.d_kv_valid) kv_valid = p.d_kv_valid[b * p.d_kv_valid_stride] + p.kv_valid_add;
  kv_valid = max(0, min(kv_valid, p.kv_max));
  const int lo = (p.window >= 0) ? max(0, kv_valid - 1 - p.window) : 0;
  int j_lo = lo / kDtKeys, j_hi = (kv_valid + kDtKeys - 1) / kDtKeys;
  {
    const int per = min(p.tiles_cap, (j_hi - j_lo + p.nsplit - 1) / p.nsplit);
    j_lo = min(j_hi, j_lo + split * per);
    j_hi = min(j_hi, j_lo + per);
  }
  const int newest = p.stable_prefix ? kv_valid - 1 : -1;   // this row comes after the wait

  const __nv_bfloat16* Qb = p.Q + ((size_t)b * p.H + (size_t)kvh * p.group) * D;
  const __nv_bfloat16* Kb = p.K + (size_t)b * p.kv_batch_stride + (size_t)kvh * p.kv_head_stride;
  const __nv_bfloat16* Vb = p.V + (size_t)b * p.kv_batch_stride + (size_t)kvh * p.kv_head_stride;

  // rows of tile j (first or second pass: all rows but `newest`, or `newest` alone); rows past the
  // key count are zero-filled
  auto load_tile = [&](int j, bool only_newest) {
    const uint32_t kt = sK + (j - j_lo) * kTile, vt = sV + (j - j_lo) * kTile;
#pragma unroll
    for (int i = 0; i < (kDtKeys * kChunks) / kDtResThreads; ++i) {
      const int idx = tid + i * kDtResThreads;
      const int r = idx / kChunks, c = idx % kChunks;
      const int row = j * kDtKeys + r;
      if ((row == newest) != only_newest) continue;
      const bool live = row < kv_valid;
      const size_t off = (size_t)(live ? row : 0) * p.kv_seq_stride + c * 8;
      dt_cp_async16(kt + dt_swz<D>(r, c), Kb + off, live);
      dt_cp_async16(vt + dt_swz<D>(r, c), Vb + off, live);
    }
  };
  for (int j = j_lo; j < j_hi; ++j) load_tile(j, false);
  dt_commit();
  if (p.stable_prefix) {
    pdl_wait();
    if (newest >= j_lo * kDtKeys && newest < j_hi * kDtKeys) load_tile(newest / kDtKeys, true);
  }
  // the query heads of this KV head are rows 0 .. group-1 of the tile; the rest are zeros
  for (int idx = tid; idx < 16 * kChunks; idx += kDtResThreads) {
    const int r = idx / kChunks, c = idx % kChunks;
    const bool live = r < p.group;
    dt_cp_async16(sQ + dt_swz<D>(r, c), Qb + (size_t)(live ? r : 0) * D + c * 8, live);
  }
  dt_commit();
  dt_wait<0>();
  __syncthreads();

  uint32_t qf[D / 16][4];
  float o[D / 8][4];
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
#pragma unroll
  for (int i = 0; i < D / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
  dt_load_q<D>(sQ, lane, qf);
  for (int j = j_lo + (warp >> 2); j < j_hi; j += 2)
    dt_tile<D>(sK + (j - j_lo) * kTile, sV + (j - j_lo) * kTile, j * kDtKeys, kv_valid, lo, p.scale_log2, warp & 3, lane,
               qf, o, m_run, l_run);
  __syncthreads();    // the partials go over the tiles

  float* part = reinterpret_cast<float*>(dt_smem);
  dt_park<D>(part, warp, lane, o, m_run, l_run);
  __syncthreads();
  const int pair = b * gridDim.x + kvh;
  float* mine = g_dt_partial + ((size_t)pair * p.nsplit + split) * 16 * kRow;
  dt_fold_warps<D, 8>(part, mine, p.group, tid, kDtResThreads);
  __syncthreads();
  if (tid == 0) {
    // release: the barrier orders the CTA's writes before this, acquire: the folding CTA's reads after it
    unsigned int old;
    asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], 1;" : "=r"(old) : "l"(&g_dt_arrived[pair]) : "memory");
    s_last = old == (unsigned)p.nsplit - 1;
  }
  __syncthreads();
  if (!s_last) return;
  // ---- the last CTA of the pair folds every CTA's partial (read past L1: other SMs wrote them).  Two round
  // trips to L2, every load of a round in flight together: the (max, sum) pairs, a warp per query head, give
  // each CTA's weight; then every thread sums its outputs over the CTAs. ----
  const float* all = g_dt_partial + (size_t)pair * p.nsplit * 16 * kRow;
  float* coef = reinterpret_cast<float*>(dt_smem);          // [group][nsplit], scaled by 1 / sum
  // the usual case (up to 20 CTAs a pair, up to two outputs a thread): the outputs' loads go out with the
  // (max, sum) loads, one round trip in all
  const bool quick = p.nsplit <= 20 && p.group * D <= 2 * kDtResThreads;
  float pre[2][20];
  if (quick) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int idx = tid + i * kDtResThreads;
      const int row = idx / D, d = idx - row * D;
#pragma unroll
      for (int u = 0; u < 20; ++u)
        pre[i][u] = (idx < p.group * D && u < p.nsplit) ? __ldcg(all + ((size_t)u * 16 + row) * kRow + d) : 0.f;
    }
  }
  constexpr int kPer = (kDtResCtas + 31) / 32;              // CTAs a lane looks at
  for (int row = warp; row < p.group; row += kDtResThreads / 32) {
    float mr[kPer], lr[kPer];
#pragma unroll
    for (int u = 0; u < kPer; ++u) {
      const int r = lane + 32 * u;
      mr[u] = -INFINITY; lr[u] = 0.f;
      if (r < p.nsplit) {
        const float2 ml = __ldcg(reinterpret_cast<const float2*>(all + ((size_t)r * 16 + row) * kRow + D));
        mr[u] = ml.x; lr[u] = ml.y;
      }
    }
    float Mx = -INFINITY;
#pragma unroll
    for (int u = 0; u < kPer; ++u) Mx = fmaxf(Mx, mr[u]);
    Mx = warp_max(Mx);
    float c[kPer], Ls = 0.f;
#pragma unroll
    for (int u = 0; u < kPer; ++u) {
      c[u] = (mr[u] == -INFINITY) ? 0.f : dt_ex2(mr[u] - Mx);
      Ls = fmaf(lr[u], c[u], Ls);
    }
    Ls = warp_sum(Ls);
    const float inv = Ls > 0.f ? 1.0f / Ls : 0.f;
#pragma unroll
    for (int u = 0; u < kPer; ++u) {
      const int r = lane + 32 * u;
      if (r < p.nsplit) coef[row * p.nsplit + r] = c[u] * inv;
    }
  }
  __syncthreads();
  if (quick) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int idx = tid + i * kDtResThreads;
      if (idx < p.group * D) {
        const int row = idx / D, d = idx - row * D;
        const float* cf = coef + row * p.nsplit;
        float acc = 0.f;
#pragma unroll
        for (int u = 0; u < 20; ++u)
          if (u < p.nsplit) acc = fmaf(pre[i][u], cf[u], acc);
        p.O[((size_t)b * p.H + (size_t)kvh * p.group + row) * D + d] = __float2bfloat16_rn(acc);
      }
    }
  }
  for (int idx = tid; idx < (quick ? 0 : p.group * D); idx += kDtResThreads) {
    const int row = idx / D, d = idx - row * D;
    const float* src = all + (size_t)row * kRow + d;
    const float* cf = coef + row * p.nsplit;
    float acc = 0.f;
    for (int r0 = 0; r0 < p.nsplit; r0 += 20) {
      float v[20];
#pragma unroll
      for (int u = 0; u < 20; ++u) v[u] = r0 + u < p.nsplit ? __ldcg(src + (size_t)(r0 + u) * 16 * kRow) : 0.f;
#pragma unroll
      for (int u = 0; u < 20; ++u)
        if (r0 + u < p.nsplit) acc = fmaf(v[u], cf[r0 + u], acc);
    }
    p.O[((size_t)b * p.H + (size_t)kvh * p.group + row) * D + d] = __float2bfloat16_rn(acc);
  }
  if (tid == 0) g_dt_arrived[pair] = 0;    // every CTA of the pair has arrived: ready for the next launch
}

template <int D>
static int launch_decode_resident(const DecodeTcParams& p, int batch, cudaStream_t stream) {
  constexpr int kTile = kDtKeys * D * 2;
  // the tiles; the eight warps' partials and the fold's weights lie over them
  int smem = 16 * D * 2 + 2 * p.tiles_cap * kTile;
  if (smem < 8 * 16 * (D + 2) * 4) smem = 8 * 16 * (D + 2) * 4;
  static DeviceOnce configured;   // the attribute is per device
  if (!configured.done()) {
    if (cudaFuncSetAttribute(mha_decode_resident_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) !=
        cudaSuccess)
      return IRON_ERR_LAUNCH;
    configured.mark();
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(p.G, batch, p.nsplit);
  cfg.blockDim = dim3(kDtResThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  fill_pdl_attr(cfg, attr);
  return cudaLaunchKernelEx(&cfg, mha_decode_resident_kernel<D>, p) == cudaSuccess ? IRON_OK : IRON_ERR_LAUNCH;
}

template <int D>
static int launch_decode_tc(const DecodeTcParams& p, int batch, cudaStream_t stream) {
  // Q tile + double-buffered K and V tiles; the merge reuses the same bytes
  constexpr int kTiles = 16 * D * 2 + 4 * kDtKeys * D * 2;
  constexpr int kMerge = 5 * 16 * (D + 2) * 4;   // the four warps' partials and the CTA's own
  constexpr int kSmem = kTiles > kMerge ? kTiles : kMerge;
  static DeviceOnce configured;   // the attribute is per device
  if (!configured.done()) {
    if (cudaFuncSetAttribute(mha_decode_tc_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem) !=
        cudaSuccess)
      return IRON_ERR_LAUNCH;
    configured.mark();
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(p.G, batch, p.nsplit);
  cfg.blockDim = dim3(kDtThreads);
  cfg.dynamicSmemBytes = kSmem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  fill_pdl_attr(cfg, attr);
  if (p.nsplit > 1) {
    cudaLaunchAttribute& c = attr[cfg.numAttrs++];
    c.id = cudaLaunchAttributeClusterDimension;
    c.val.clusterDim.x = 1;
    c.val.clusterDim.y = 1;
    c.val.clusterDim.z = p.nsplit;
  }
  return cudaLaunchKernelEx(&cfg, mha_decode_tc_kernel<D>, p) == cudaSuccess ? IRON_OK : IRON_ERR_LAUNCH;
}

// Called by iron_mha_decode_bf16 for a few sequences: the resident form.  IRON_ERR_UNSUPPORTED when a CTA's
// share of the longest cache does not fit its shared memory (the caller takes the streaming kernels).
int mha_decode_resident(const void* Q, const void* K, const void* V, void* O, int batch, int H, int G, int D,
                        int kv_max, long long kv_batch_stride, long long kv_seq_stride, long long kv_head_stride,
                        int kv_valid, const int* d_kv_valid, int d_kv_valid_stride, int kv_valid_add, int window,
                        float scale, int stable_prefix, cudaStream_t stream) {
  const int group = H / G, pairs = batch * G;
  if (group > 16 || (D != 64 && D != 128) || pairs > kDtResPairs || pairs > kSMs) return IRON_ERR_UNSUPPORTED;
  const int tiles = (kv_max + kDtKeys - 1) / kDtKeys;
  int nsplit = kSMs / pairs;
  if (nsplit > 20) nsplit = 20;       // the last CTA folds up to 20 partials in one round trip
  if (nsplit > tiles) nsplit = tiles;
  if (nsplit < 1 || pairs * nsplit > kDtResCtas) return IRON_ERR_UNSUPPORTED;
  const int tiles_cap = (tiles + nsplit - 1) / nsplit;
  if (16 * D * 2 + 2 * tiles_cap * kDtKeys * D * 2 > 200 * 1024) return IRON_ERR_UNSUPPORTED;
  DecodeTcParams p = {};
  p.Q = (const __nv_bfloat16*)Q; p.K = (const __nv_bfloat16*)K; p.V = (const __nv_bfloat16*)V;
  p.O = (__nv_bfloat16*)O;
  p.kv_batch_stride = kv_batch_stride; p.kv_seq_stride = kv_seq_stride; p.kv_head_stride = kv_head_stride;
  p.H = H; p.G = G; p.group = group;
  p.kv_valid = kv_valid; p.d_kv_valid = d_kv_valid; p.d_kv_valid_stride = d_kv_valid_stride;
  p.kv_valid_add = kv_valid_add; p.kv_max = kv_max; p.window = window;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.nsplit = nsplit; p.tiles_cap = tiles_cap; p.stable_prefix = stable_prefix;
  return D == 64 ? launch_decode_resident<64>(p, batch, stream) : launch_decode_resident<128>(p, batch, stream);
}

// Called by iron_mha_decode_bf16 for batches that fill the machine; the arguments are that
// entry point's, already validated.  Returns IRON_ERR_UNSUPPORTED when the shape is not
// this kernel's (the caller then takes the SIMT kernel).
int mha_decode_tc(const void* Q, const void* K, const void* V, void* O, int batch, int H, int G, int D, int kv_max,
                  long long kv_batch_stride, long long kv_seq_stride, long long kv_head_stride, int kv_valid,
                  const int* d_kv_valid, int d_kv_valid_stride, int kv_valid_add, int window, float scale,
                  cudaStream_t stream) {
  const int group = H / G;
  if (group > 16 || (D != 64 && D != 128)) return IRON_ERR_UNSUPPORTED;
  DecodeTcParams p = {};
  p.Q = (const __nv_bfloat16*)Q; p.K = (const __nv_bfloat16*)K; p.V = (const __nv_bfloat16*)V;
  p.O = (__nv_bfloat16*)O;
  p.kv_batch_stride = kv_batch_stride; p.kv_seq_stride = kv_seq_stride; p.kv_head_stride = kv_head_stride;
  p.H = H; p.G = G; p.group = group;
  p.kv_valid = kv_valid; p.d_kv_valid = d_kv_valid; p.d_kv_valid_stride = d_kv_valid_stride;
  p.kv_valid_add = kv_valid_add; p.kv_max = kv_max; p.window = window;
  p.scale_log2 = scale * 1.4426950408889634f;
  // split the keys while the machine is not yet full and a CTA keeps at least four tiles of the longest run
  p.nsplit = 1;
  const int tiles = (kv_max + kDtKeys - 1) / kDtKeys;
  // (up to two CTAs an SM: one an SM and four an SM both measured slower on 4 to 16 sequences of 4096 keys)
  while (p.nsplit < 8 && (long long)batch * G * p.nsplit * 2 <= 2 * kSMs && tiles / (p.nsplit * 2) >= 4) p.nsplit *= 2;
  return D == 64 ? launch_decode_tc<64>(p, batch, stream) : launch_decode_tc<128>(p, batch, stream);
}

}  // namespace iron
