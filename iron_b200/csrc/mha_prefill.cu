// Multi-query ("prompt chunk") attention with grouped-query heads: causal, windowed or
// bidirectional, the queries being the last rows of the keys.
//
// One CTA = 64 query rows of one head (4 warps x 16 rows); keys and values stream
// through shared memory in 64-row tiles (cp.async, double buffered, 16-byte chunks
// XOR-swizzled so ldmatrix is conflict-free).  S = Q K^T and O += P V run on the warp
// MMA (m16n8k16, bf16 in, f32 out) with the online softmax in registers, exp2 domain.
// Key blocks wholly above the causal diagonal or below the window are skipped, so the
// work follows the context.  Rows past the call's bound are written as zeros and keys
// past its bound are masked, as the reference's bounded call does.
#include <cstdlib>

#include "common.cuh"

namespace iron {

struct PrefillParams {
  const __nv_bfloat16* Q;
  const __nv_bfloat16* K;
  const __nv_bfloat16* V;
  __nv_bfloat16* O;
  long long q_batch_stride, q_row_stride, q_head_stride;     // elements
  long long o_batch_stride, o_row_stride, o_head_stride;     // elements
  long long kv_batch_stride, kv_row_stride, kv_head_stride;  // elements
  int H, G;
  int q_rows;       // rows of Q and O (written: the bound's rows computed, the rest zero)
  int kv_rows;      // rows of K and V
  int q_tokens;     // the call's query bound
  const int* d_q_tokens;
  int kv_tokens;    // the call's key bound; the queries are its last q_tokens rows
  const int* d_kv_tokens;
  int kv_tokens_add;
  int causal;
  int window;       // < 0: none
  float scale_log2;
};

constexpr int kPfThreads = 128;
constexpr int kBlockM = 64;
constexpr int kBlockN = 64;

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool pred) {
  const int bytes = pred ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// 2^x on the special-function unit, one instruction (no denormal rescue: a probability
// below 2^-126 is zero either way once it is rounded to bf16).
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Byte offset of 16-byte chunk `chunk` of row `row` in a tile whose rows are D bf16 wide.
template <int D>
__device__ __forceinline__ uint32_t swz(int row, int chunk) {
  return (uint32_t)(row * (D * 2) + ((((chunk & 7) ^ (row & 7)) | (chunk & ~7)) << 4));
}

// Copy rows [row0, row0 + 64) x D of a strided matrix into a swizzled tile; rows >= limit zero.
template <int D>
__device__ __forceinline__ void load_tile(uint32_t smem_tile, const __nv_bfloat16* base, long long row_stride,
                                          int row0, int limit, int tid) {
  constexpr int kChunks = D / 8;
#pragma unroll
  for (int i = 0; i < (kBlockN * kChunks) / kPfThreads; ++i) {
    const int idx = tid + i * kPfThreads;
    const int r = idx / kChunks, c = idx % kChunks;
    const bool live = row0 + r < limit;
    const __nv_bfloat16* src = base + (long long)(live ? row0 + r : 0) * row_stride + c * 8;
    cp_async16(smem_tile + swz<D>(r, c), src, live);
  }
}

// MT: 16-row query tiles per warp.  With MT = 2 a CTA covers 128 query rows and every K and V
// fragment read from shared memory feeds two MMAs.
template <int D, int MT>
__global__ void __launch_bounds__(kPfThreads) mha_prefill_kernel(const PrefillParams p) {
  extern __shared__ __align__(128) uint8_t pf_smem[];
  constexpr int kTile = kBlockN * D * 2;
  constexpr int kRowsM = kBlockM * MT;          // query rows of a CTA
  const uint32_t sQ = smem_u32(pf_smem);
  const uint32_t sK = sQ + MT * kTile, sV = sK + 2 * kTile;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int head = blockIdx.x, b = blockIdx.z;
  const int kvh = head / (p.H / p.G);

  pdl_wait();
  pdl_launch();

  int q_tokens = p.d_q_tokens ? *p.d_q_tokens : p.q_tokens;
  q_tokens = max(0, min(q_tokens, p.q_rows));
  int kv_tokens = p.d_kv_tokens ? (*p.d_kv_tokens + p.kv_tokens_add) : p.kv_tokens;
  kv_tokens = max(0, min(kv_tokens, p.kv_rows));
  const bool masked = p.causal || p.window >= 0;
  const int offset = masked ? kv_tokens - q_tokens : 0;  // position of query row 0

  // Heavy (late) query blocks first, for every head, before any light one: the heads are
  // the fast grid dimension, so the tail of the launch is made of the shortest key ranges.
  const int qb = gridDim.y - 1 - blockIdx.y;
  const int m0 = qb * kRowsM;
  __nv_bfloat16* Ob = p.O + (long long)b * p.o_batch_stride + (long long)head * p.o_head_stride;

  if (m0 >= q_tokens || offset < 0 || kv_tokens == 0) {
    // nothing to attend from: the block's rows are zeros
    for (int idx = tid; idx < kRowsM * (D / 8); idx += kPfThreads) {
      const int r = idx / (D / 8), c = idx % (D / 8);
      if (m0 + r < p.q_rows)
        *reinterpret_cast<uint4*>(Ob + (long long)(m0 + r) * p.o_row_stride + c * 8) = make_uint4(0, 0, 0, 0);
    }
    return;
  }

  const __nv_bfloat16* Qb = p.Q + (long long)b * p.q_batch_stride + (long long)head * p.q_head_stride;
  const __nv_bfloat16* Kb = p.K + (long long)b * p.kv_batch_stride + (long long)kvh * p.kv_head_stride;
  const __nv_bfloat16* Vb = p.V + (long long)b * p.kv_batch_stride + (long long)kvh * p.kv_head_stride;

  // key blocks this query block can see
  int j_lo = 0, j_hi = (kv_tokens + kBlockN - 1) / kBlockN;
  if (p.causal) j_hi = min(j_hi, (offset + min(m0 + kRowsM, q_tokens) - 1) / kBlockN + 1);
  else if (p.window >= 0) j_hi = min(j_hi, (offset + min(m0 + kRowsM, q_tokens) - 1 + p.window) / kBlockN + 1);
  if (p.window >= 0) j_lo = max(0, (offset + m0 - p.window) / kBlockN);

#pragma unroll
  for (int mt = 0; mt < MT; ++mt) load_tile<D>(sQ + mt * kTile, Qb, p.q_row_stride, m0 + mt * kBlockM, q_tokens, tid);
  load_tile<D>(sK, Kb, p.kv_row_stride, j_lo * kBlockN, kv_tokens, tid);
  load_tile<D>(sV, Vb, p.kv_row_stride, j_lo * kBlockN, kv_tokens, tid);
  cp_async_commit();

  // query tile mt of this warp: rows m0 + mt * 64 + warp * 16 ..+ 16
  uint32_t qf[MT][D / 16][4];
  float o[MT][D / 8][4];
  float m_run[MT][2], l_run[MT][2];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) {
    m_run[mt][0] = m_run[mt][1] = -INFINITY;
    l_run[mt][0] = l_run[mt][1] = 0.f;
#pragma unroll
    for (int i = 0; i < D / 8; ++i) { o[mt][i][0] = o[mt][i][1] = o[mt][i][2] = o[mt][i][3] = 0.f; }
  }

  for (int j = j_lo; j < j_hi; ++j) {
    const int buf = (j - j_lo) & 1;
    if (j + 1 < j_hi) {  // prefetch the next key/value tiles into the other buffer
      load_tile<D>(sK + (buf ^ 1) * kTile, Kb, p.kv_row_stride, (j + 1) * kBlockN, kv_tokens, tid);
      load_tile<D>(sV + (buf ^ 1) * kTile, Vb, p.kv_row_stride, (j + 1) * kBlockN, kv_tokens, tid);
    }
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();

    if (j == j_lo) {
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
        for (int kt = 0; kt < D / 16; ++kt) {
          const int row = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
          ldmatrix_x4(sQ + mt * kTile + swz<D>(row, kt * 2 + (lane >> 4)), qf[mt][kt][0], qf[mt][kt][1],
                      qf[mt][kt][2], qf[mt][kt][3]);
        }
      }
    }
    const int key0 = j * kBlockN;
    // a query tile whose rows all sit above this key block has nothing to do here (causal)
    bool dead[MT];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
      dead[mt] = p.causal && key0 > offset + m0 + mt * kBlockM + warp * 16 + 15;

    // ---- S = Q K^T (16 x 64 per query tile) ----
    float s[MT][kBlockN / 8][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
      for (int nt = 0; nt < kBlockN / 8; ++nt) { s[mt][nt][0] = s[mt][nt][1] = s[mt][nt][2] = s[mt][nt][3] = 0.f; }
    }
    const uint32_t kt_base = sK + buf * kTile;
#pragma unroll
    for (int kt = 0; kt < D / 16; ++kt) {
#pragma unroll
      for (int np = 0; np < kBlockN / 16; ++np) {
        uint32_t b0, b1, b2, b3;
        const int row = np * 16 + (lane & 7) + (lane >> 4) * 8;
        ldmatrix_x4(kt_base + swz<D>(row, kt * 2 + ((lane >> 3) & 1)), b0, b1, b2, b3);
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          if (dead[mt]) continue;
          mma_bf16(s[mt][2 * np], qf[mt][kt], b0, b1);
          mma_bf16(s[mt][2 * np + 1], qf[mt][kt], b2, b3);
        }
      }
    }

    // ---- scale, mask, online softmax ----
    uint32_t pf[MT][kBlockN / 16][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
      if (dead[mt]) continue;
      const int row_a = m0 + mt * kBlockM + warp * 16 + g;  // this thread's rows: row_a and row_a + 8
      const bool partial = (key0 + kBlockN > kv_tokens) || p.window >= 0 ||
                           (p.causal && key0 + kBlockN - 1 > offset + m0 + mt * kBlockM + warp * 16);
      float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int nt = 0; nt < kBlockN / 8; ++nt) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float v = s[mt][nt][e] * p.scale_log2;
          if (partial) {
            const int key = key0 + nt * 8 + 2 * t + (e & 1);
            const int pos = offset + row_a + (e >> 1) * 8;
            bool ok = key < kv_tokens;
            if (p.causal) ok = ok && key <= pos;
            else if (p.window >= 0) ok = ok && key <= pos + p.window;
            if (p.window >= 0) ok = ok && key >= pos - p.window;
            if (!ok) v = -INFINITY;
          }
          s[mt][nt][e] = v;
          mx[e >> 1] = fmaxf(mx[e >> 1], v);
        }
      }
      float corr[2], msafe[2];
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
        const float mn = fmaxf(m_run[mt][r], mx[r]);
        msafe[r] = (mn == -INFINITY) ? 0.f : mn;
        corr[r] = ex2(m_run[mt][r] - msafe[r]);  // m_run = -inf gives 0
        m_run[mt][r] = mn;
        l_run[mt][r] *= corr[r];
      }
      float ls[2] = {0.f, 0.f};
#pragma unroll
      for (int nt = 0; nt < kBlockN / 8; ++nt) {
        const float p0 = ex2(s[mt][nt][0] - msafe[0]), p1 = ex2(s[mt][nt][1] - msafe[0]);
        const float p2 = ex2(s[mt][nt][2] - msafe[1]), p3 = ex2(s[mt][nt][3] - msafe[1]);
        ls[0] += p0 + p1;
        ls[1] += p2 + p3;
        pf[mt][nt >> 1][(nt & 1) * 2] = pack_bf16x2(p0, p1);
        pf[mt][nt >> 1][(nt & 1) * 2 + 1] = pack_bf16x2(p2, p3);
      }
      l_run[mt][0] += ls[0];
      l_run[mt][1] += ls[1];
#pragma unroll
      for (int dt = 0; dt < D / 8; ++dt) {
        o[mt][dt][0] *= corr[0]; o[mt][dt][1] *= corr[0];
        o[mt][dt][2] *= corr[1]; o[mt][dt][3] *= corr[1];
      }
    }

    // ---- O += P V ----
    const uint32_t vt_base = sV + buf * kTile;
#pragma unroll
    for (int kt2 = 0; kt2 < kBlockN / 16; ++kt2) {
#pragma unroll
      for (int dp = 0; dp < D / 16; ++dp) {
        uint32_t b0, b1, b2, b3;
        const int row = kt2 * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
        ldmatrix_x4_trans(vt_base + swz<D>(row, dp * 2 + (lane >> 4)), b0, b1, b2, b3);
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          if (dead[mt]) continue;
          mma_bf16(o[mt][2 * dp], pf[mt][kt2], b0, b1);
          mma_bf16(o[mt][2 * dp + 1], pf[mt][kt2], b2, b3);
        }
      }
    }
    __syncthreads();  // the other buffer is overwritten by the next iteration's prefetch
  }
  cp_async_wait<0>();

  // ---- normalise and store; rows past the bound are zeros ----
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      float l = l_run[mt][r];
      l += __shfl_xor_sync(0xffffffffu, l, 1);
      l += __shfl_xor_sync(0xffffffffu, l, 2);
      const int row = m0 + mt * kBlockM + warp * 16 + g + r * 8;
      if (row >= p.q_rows) continue;
      const bool live = row < q_tokens;
      const float inv = (live && l > 0.f) ? 1.0f / l : 0.f;
      __nv_bfloat16* dst = Ob + (long long)row * p.o_row_stride;
#pragma unroll
      for (int dt = 0; dt < D / 8; ++dt)
        *reinterpret_cast<uint32_t*>(dst + dt * 8 + 2 * t) =
            pack_bf16x2(o[mt][dt][2 * r] * inv, o[mt][dt][2 * r + 1] * inv);
    }
  }
}

template <int D, int MT>
static int launch_prefill(const PrefillParams& p, int batch, cudaStream_t stream) {
  constexpr int kSmem = (MT + 4) * kBlockN * D * 2;
  static DeviceOnce configured;   // the attribute is per device
  if (!configured.done()) {
    if (cudaFuncSetAttribute(mha_prefill_kernel<D, MT>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem) !=
        cudaSuccess)
      return IRON_ERR_LAUNCH;
    configured.mark();
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(p.H, (p.q_rows + kBlockM * MT - 1) / (kBlockM * MT), batch);
  cfg.blockDim = dim3(kPfThreads);
  cfg.dynamicSmemBytes = kSmem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  fill_pdl_attr(cfg, attr);
  return cudaLaunchKernelEx(&cfg, mha_prefill_kernel<D, MT>, p) == cudaSuccess ? IRON_OK : IRON_ERR_LAUNCH;
}

// mha_prefill_tc.cu
int mha_prefill_tc(const void* Q, const void* K, const void* V, void* O, int batch, int H, int G, int D,
                   int q_rows, long long q_batch_stride, long long q_row_stride, long long q_head_stride,
                   long long o_batch_stride, long long o_row_stride, long long o_head_stride,
                   long long kv_batch_stride, long long kv_row_stride, long long kv_head_stride, int q_tokens,
                   int kv_tokens, int causal, int window, float scale, int* d_status, cudaStream_t stream);

}  // namespace iron

using namespace iron;

static int* g_prefill_status[64] = {};   // one status word per device

extern "C" void iron_mha_prefill_status_word(int* d_status) {
  const int dev = current_device();
  if (dev >= 0) g_prefill_status[dev] = d_status;
}

extern "C" int iron_mha_prefill_bf16(const void* Q, const void* K, const void* V, void* O, int batch, int H,
                                     int G, int D, int q_rows, int kv_rows, long long q_batch_stride,
                                     long long q_row_stride, long long q_head_stride,
                                     long long o_batch_stride, long long o_row_stride,
                                     long long o_head_stride, long long kv_batch_stride, long long kv_row_stride,
                                     long long kv_head_stride, int q_tokens, const int* d_q_tokens,
                                     int kv_tokens, const int* d_kv_tokens, int kv_tokens_add, int causal,
                                     int window, float scale, iron_stream_t stream) {
  if (batch <= 0 || H <= 0 || G <= 0 || H % G) return IRON_ERR_SHAPE;
  if (D != 64 && D != 128) return IRON_ERR_SHAPE;
  if (q_rows <= 0 || kv_rows <= 0) return IRON_ERR_SHAPE;
  if (q_tokens < 0 || q_tokens > q_rows || kv_tokens < 0 || kv_tokens > kv_rows) return IRON_ERR_SHAPE;
  if ((causal || window >= 0) && !d_q_tokens && !d_kv_tokens && kv_tokens < q_tokens) return IRON_ERR_SHAPE;
  if ((o_row_stride & 7) || (o_head_stride & 7) || (o_batch_stride & 7)) return IRON_ERR_ALIGN;
  if ((q_row_stride & 7) || (q_head_stride & 7) || (q_batch_stride & 7) || (kv_row_stride & 7) ||
      (kv_head_stride & 7) || (kv_batch_stride & 7))
    return IRON_ERR_ALIGN;
  if (!aligned16(Q) || !aligned16(K) || !aligned16(V) || !aligned16(O)) return IRON_ERR_ALIGN;
  PrefillParams p = {};
  p.Q = (const __nv_bfloat16*)Q; p.K = (const __nv_bfloat16*)K; p.V = (const __nv_bfloat16*)V;
  p.O = (__nv_bfloat16*)O;
  p.q_batch_stride = q_batch_stride; p.q_row_stride = q_row_stride; p.q_head_stride = q_head_stride;
  p.o_batch_stride = o_batch_stride; p.o_row_stride = o_row_stride; p.o_head_stride = o_head_stride;
  p.kv_batch_stride = kv_batch_stride; p.kv_row_stride = kv_row_stride; p.kv_head_stride = kv_head_stride;
  p.H = H; p.G = G; p.q_rows = q_rows; p.kv_rows = kv_rows;
  p.q_tokens = q_tokens; p.d_q_tokens = d_q_tokens;
  p.kv_tokens = kv_tokens; p.d_kv_tokens = d_kv_tokens; p.kv_tokens_add = kv_tokens_add;
  p.causal = causal; p.window = window;
  p.scale_log2 = scale * 1.4426950408889634f;
  cudaStream_t s = (cudaStream_t)stream;
  // Bounds known on the host and at least a tile of queries: the tensor-memory kernel
  // (IRON_MHA_PREFILL_TC=0 keeps the warp-MMA kernel).
  if (!d_q_tokens && !d_kv_tokens && q_tokens >= 128) {
    const char* e = getenv("IRON_MHA_PREFILL_TC");
    if (!(e && e[0] == '0')) {
      const int rc = mha_prefill_tc(Q, K, V, O, batch, H, G, D, q_rows, q_batch_stride, q_row_stride, q_head_stride,
                                    o_batch_stride, o_row_stride, o_head_stride, kv_batch_stride, kv_row_stride,
                                    kv_head_stride, q_tokens, kv_tokens, causal, window, scale, current_device() >= 0 ? g_prefill_status[current_device()] : nullptr, s);
      if (rc != IRON_ERR_UNSUPPORTED) return rc;
    }
  }
  // One 16-row query tile per warp: two (128 query rows per CTA, every K/V fragment feeding
  // two MMAs) measured slower at 2048 x 2048 -- 249 registers leave 8 warps per SM.
  if (D == 64) return launch_prefill<64, 1>(p, batch, s);
  return launch_prefill<128, 1>(p, batch, s);
}
