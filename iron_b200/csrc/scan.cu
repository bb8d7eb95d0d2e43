// Mamba2: the selective-scan recurrence and the short causal depth-wise convolution.
//
// Selective scan.  The recurrence is sequential in time and independent over
// (batch, head, head_dim row); float32 throughout, y rounded once, as the reference's.
// A CTA of 128 threads owns one head and up to 64 rows of its (head_dim x state_size)
// state: thread (p, half) keeps half of row p's state in registers (packed f32x2
// arithmetic), so a time step costs two packed FMAs and one packed multiply per state
// pair and a single shuffle per row -- no cross-lane reduction tree.  The step's B, C,
// x and dt are staged 16 time steps at a time through shared memory (converted to f32
// once per CTA, the next block's global loads in flight while the current block
// computes), and y leaves through a shared tile so stores are 128-byte rows.
//
// Causal conv.  y[t] = sum_k taps[k] * x[t - K + 1 + k] per channel, the K - 1 rows before
// the call read from a history buffer, with the reference's operator chain roundings
// (each product and each partial sum rounded to bf16), optional bias and SiLU fused.
#include "common.cuh"
#include "mma.cuh"
#include "scan.cuh"

namespace iron {

constexpr int kScanThreads = 128;
constexpr int kTB = 16;   // time steps staged per block

// TPP threads share a pair of state rows (4 or 8); a CTA covers kPT = 2 * 128 / TPP rows of a head.
template <int N, int TPP>
__global__ void __launch_bounds__(kScanThreads) selective_scan_kernel(const ScanParams p) {
  constexpr int kPT = 2 * (kScanThreads / TPP);   // head_dim rows per CTA
  constexpr int NQ = N / (4 * TPP);               // float4 groups of states per thread and row
  constexpr int CB = N / 8;        // 16-byte chunks per B (or C) row
  constexpr int kBC = (kTB * CB + kScanThreads - 1) / kScanThreads;  // chunks per thread per block
  __shared__ __align__(16) float sB[2][kTB][N];
  __shared__ __align__(16) float sC[2][kTB][N];
  __shared__ __align__(16) float sX[2][kTB][kPT];
  __shared__ float2 sDt[2][kTB];   // (step, exp(step * A))
  __shared__ __align__(16) __nv_bfloat16 sY[kTB][kPT];

  // A thread owns two state rows (2 rp, 2 rp + 1) and every TPP-th float4 group of N:
  // B and C, which all rows of a head share, are read from shared memory once for both
  // rows, and the TPP threads of a row pair read one contiguous run (no bank conflict).
  const int tid = threadIdx.x, rp = tid / TPP, q = tid % TPP;
  const int ptiles = (p.P + kPT - 1) / kPT;
  const int h = blockIdx.x / ptiles, p0 = (blockIdx.x - h * ptiles) * kPT;
  const int b = blockIdx.y;
  const int grp = h / (p.H / p.G);
  const int pcount = min(kPT, p.P - p0);
  const bool live_a = 2 * rp < pcount, live_b = 2 * rp + 1 < pcount;
  const int inner = p.H * p.P;

  pdl_wait();
  pdl_launch();
  int valid = p.d_valid ? min(*p.d_valid, p.rows) : p.valid;
  valid = max(valid, 0);

  const float dt_bias = p.head[h * 3], A = p.head[h * 3 + 1], Dh = p.head[h * 3 + 2];
  const __nv_bfloat16* xbc = p.xbc + (size_t)b * p.xbc_batch;
  const __nv_bfloat16* dtp = p.dt + (size_t)b * p.dt_batch;
  __nv_bfloat16* yb = p.y + (size_t)b * p.y_batch;

  float2 sa[2 * NQ], sb[2 * NQ];   // group j of this thread: states (4 j + q) * 4 .. + 4
#pragma unroll
  for (int i = 0; i < 2 * NQ; ++i) { sa[i] = make_float2(0.f, 0.f); sb[i] = make_float2(0.f, 0.f); }
  if (p.state) {
    const float* src = p.state + (size_t)b * p.state_batch + ((size_t)h * p.P + p0 + 2 * rp) * N;
#pragma unroll
    for (int j = 0; j < NQ; ++j) {
      const int n0 = (TPP * j + q) * 4;
      if (live_a) {
        const float4 v = *reinterpret_cast<const float4*>(src + n0);
        sa[2 * j] = make_float2(v.x, v.y); sa[2 * j + 1] = make_float2(v.z, v.w);
      }
      if (live_b) {
        const float4 v = *reinterpret_cast<const float4*>(src + N + n0);
        sb[2 * j] = make_float2(v.x, v.y); sb[2 * j + 1] = make_float2(v.z, v.w);
      }
    }
  }

  // registers holding the next block's raw rows while the current block computes
  uint4 rB[kBC], rC[kBC], rX;
  float rDt = 0.f;
  auto fetch = [&](int t0) {
#pragma unroll
    for (int i = 0; i < kBC; ++i) {
      const int idx = tid + i * kScanThreads;
      const int tt = idx / CB, c = idx - tt * CB;
      rB[i] = make_uint4(0, 0, 0, 0); rC[i] = make_uint4(0, 0, 0, 0);
      if (idx < kTB * CB && t0 + tt < valid) {
        const __nv_bfloat16* row = xbc + (size_t)(t0 + tt) * p.width + inner;
        rB[i] = ld_cached(row + (size_t)grp * N + c * 8);
        rC[i] = ld_cached(row + (size_t)(p.G + grp) * N + c * 8);
      }
    }
    {
      const int tt = tid >> 3, c = tid & 7;  // 16 steps x 8 chunks of 8 rows
      rX = make_uint4(0, 0, 0, 0);
      if (t0 + tt < valid && c * 8 < pcount) {
        const __nv_bfloat16* src = xbc + (size_t)(t0 + tt) * p.width + (size_t)h * p.P + p0 + c * 8;
        if (c * 8 + 8 <= pcount && (((p.width | (h * p.P + p0)) & 7) == 0)) {
          rX = ld_cached(src);
        } else {
          uint16_t e[8] = {0, 0, 0, 0, 0, 0, 0, 0};
          for (int j = 0; j < 8 && c * 8 + j < pcount; ++j) e[j] = __bfloat16_as_ushort(src[j]);
          rX = make_uint4(e[0] | (e[1] << 16), e[2] | (e[3] << 16), e[4] | (e[5] << 16), e[6] | (e[7] << 16));
        }
      }
    }
    if (tid < kTB) rDt = (t0 + tid < valid) ? __bfloat162float(dtp[(size_t)(t0 + tid) * p.H + h]) : 0.f;
  };
  auto stage = [&](int buf) {
#pragma unroll
    for (int i = 0; i < kBC; ++i) {
      const int idx = tid + i * kScanThreads;
      if (idx < kTB * CB) {
        const int tt = idx / CB, c = idx - tt * CB;
        float f[8];
        unpack8(rB[i], f);
        *reinterpret_cast<float4*>(&sB[buf][tt][c * 8]) = make_float4(f[0], f[1], f[2], f[3]);
        *reinterpret_cast<float4*>(&sB[buf][tt][c * 8 + 4]) = make_float4(f[4], f[5], f[6], f[7]);
        unpack8(rC[i], f);
        *reinterpret_cast<float4*>(&sC[buf][tt][c * 8]) = make_float4(f[0], f[1], f[2], f[3]);
        *reinterpret_cast<float4*>(&sC[buf][tt][c * 8 + 4]) = make_float4(f[4], f[5], f[6], f[7]);
      }
    }
    {
      const int tt = tid >> 3, c = tid & 7;
      float f[8];
      unpack8(rX, f);
      if (c * 8 < kPT) {
        *reinterpret_cast<float4*>(&sX[buf][tt][c * 8]) = make_float4(f[0], f[1], f[2], f[3]);
        *reinterpret_cast<float4*>(&sX[buf][tt][c * 8 + 4]) = make_float4(f[4], f[5], f[6], f[7]);
      }
    }
    if (tid < kTB) {
      const float step = softplus_f32(rDt + dt_bias);
      sDt[buf][tid] = make_float2(step, expf(step * A));
    }
  };

  fetch(0);
  stage(0);
  __syncthreads();

  for (int t0 = 0, blk = 0; t0 < p.rows; t0 += kTB, ++blk) {
    const int buf = blk & 1;
    const bool more = t0 + kTB < valid;
    if (more) fetch(t0 + kTB);
    const int steps = min(kTB, valid - t0);  // <= 0 past the bound: rows of zeros
    for (int tt = 0; tt < kTB; ++tt) {
      float ya = 0.f, yb2 = 0.f;
      if (tt < steps) {
        const float2 sd = sDt[buf][tt];
        const float2 xv = *reinterpret_cast<const float2*>(&sX[buf][tt][2 * rp]);
        const float2 dA2 = make_float2(sd.y, sd.y);
        const float2 xa2 = make_float2(sd.x * xv.x, sd.x * xv.x), xb2 = make_float2(sd.x * xv.y, sd.x * xv.y);
        float2 acc_a0 = make_float2(0.f, 0.f), acc_a1 = acc_a0, acc_b0 = acc_a0, acc_b1 = acc_a0;
        const float4* Bp = reinterpret_cast<const float4*>(&sB[buf][tt][0]) + q;
        const float4* Cp = reinterpret_cast<const float4*>(&sC[buf][tt][0]) + q;
#pragma unroll
        for (int j = 0; j < NQ; ++j) {
          const float4 bv = Bp[TPP * j], cv = Cp[TPP * j];
          const float2 b0 = make_float2(bv.x, bv.y), b1 = make_float2(bv.z, bv.w);
          const float2 c0 = make_float2(cv.x, cv.y), c1 = make_float2(cv.z, cv.w);
          sa[2 * j] = __ffma2_rn(dA2, sa[2 * j], __fmul2_rn(xa2, b0));
          sa[2 * j + 1] = __ffma2_rn(dA2, sa[2 * j + 1], __fmul2_rn(xa2, b1));
          sb[2 * j] = __ffma2_rn(dA2, sb[2 * j], __fmul2_rn(xb2, b0));
          sb[2 * j + 1] = __ffma2_rn(dA2, sb[2 * j + 1], __fmul2_rn(xb2, b1));
          acc_a0 = __ffma2_rn(sa[2 * j], c0, acc_a0);
          acc_a1 = __ffma2_rn(sa[2 * j + 1], c1, acc_a1);
          acc_b0 = __ffma2_rn(sb[2 * j], c0, acc_b0);
          acc_b1 = __ffma2_rn(sb[2 * j + 1], c1, acc_b1);
        }
        ya = (acc_a0.x + acc_a0.y) + (acc_a1.x + acc_a1.y);
        yb2 = (acc_b0.x + acc_b0.y) + (acc_b1.x + acc_b1.y);
#pragma unroll
        for (int off = 1; off < TPP; off <<= 1) {
          ya += __shfl_xor_sync(0xffffffffu, ya, off);
          yb2 += __shfl_xor_sync(0xffffffffu, yb2, off);
        }
        ya = fmaf(Dh, xv.x, ya);
        yb2 = fmaf(Dh, xv.y, yb2);
      } else {
#pragma unroll
        for (int off = 1; off < TPP; off <<= 1) {
          (void)__shfl_xor_sync(0xffffffffu, ya, off);
          (void)__shfl_xor_sync(0xffffffffu, yb2, off);
        }
      }
      if (q == 0)
        *reinterpret_cast<__nv_bfloat162*>(&sY[tt][2 * rp]) =
            __halves2bfloat162(__float2bfloat16_rn(ya), __float2bfloat16_rn(yb2));
    }
    __syncthreads();
    // y tile out: 16 rows x up to 64 columns
    {
      const int tt = tid >> 3, c = tid & 7;
      if (t0 + tt < p.rows && c * 8 < pcount) {
        __nv_bfloat16* dst = yb + (size_t)(t0 + tt) * inner + (size_t)h * p.P + p0 + c * 8;
        if (c * 8 + 8 <= pcount && ((inner | (h * p.P + p0)) & 7) == 0) {
          *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(&sY[tt][c * 8]);
        } else {
          for (int j = 0; j < 8 && c * 8 + j < pcount; ++j) dst[j] = sY[tt][c * 8 + j];
        }
      }
    }
    if (more) stage(buf ^ 1);
    __syncthreads();
  }

  if (p.final_state) {
    float* dst = p.final_state + (size_t)b * p.state_batch + ((size_t)h * p.P + p0 + 2 * rp) * N;
#pragma unroll
    for (int j = 0; j < NQ; ++j) {
      const int n0 = (TPP * j + q) * 4;
      if (live_a) *reinterpret_cast<float4*>(dst + n0) = make_float4(sa[2 * j].x, sa[2 * j].y, sa[2 * j + 1].x, sa[2 * j + 1].y);
      if (live_b)
        *reinterpret_cast<float4*>(dst + N + n0) = make_float4(sb[2 * j].x, sb[2 * j].y, sb[2 * j + 1].x, sb[2 * j + 1].y);
    }
  }
}

// ---------------------------------------------------------------- causal conv
struct ConvParams {
  const __nv_bfloat16* x;        // (B, rows, C)
  const __nv_bfloat16* taps;     // (K, C)
  const __nv_bfloat16* bias;     // (C) or null
  const __nv_bfloat16* history;  // (B, K-1, C) or null: zeros
  __nv_bfloat16* new_history;    // (B, K-1, C) or null
  __nv_bfloat16* y;              // (B, rows, C)
  int rows, C, K;
  int valid;
  const int* d_valid;
  int decode_order;              // sum the newest tap first (the one-row form's order)
  int silu;
  long long x_batch, y_batch, hist_batch;
};

// One thread per 8 channels, marching down the rows with the last K-1 inputs in registers.
//
// The recorded chain rounds every product and every sum to bf16.  A bf16 x bf16 product is
// exact in f32, and the f32 sum of two bf16 values is either exact or differs from the larger
// operand by less than 2^-16 of it, so "f32 operation, then round to bf16" is the correctly
// rounded bf16 operation: the chain runs on packed bf16x2 multiplies and adds (mul.rn.bf16x2,
// add.rn.bf16x2), two channels per instruction, bit for bit the same.
__device__ __forceinline__ uint32_t bmul2(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
__device__ __forceinline__ uint32_t badd2(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("add.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
__device__ __forceinline__ uint4 bmul8(const uint4& a, const uint4& b) {
  return make_uint4(bmul2(a.x, b.x), bmul2(a.y, b.y), bmul2(a.z, b.z), bmul2(a.w, b.w));
}
__device__ __forceinline__ uint4 badd8(const uint4& a, const uint4& b) {
  return make_uint4(badd2(a.x, b.x), badd2(a.y, b.y), badd2(a.z, b.z), badd2(a.w, b.w));
}

template <int K>
__global__ void __launch_bounds__(128) causal_conv_kernel(const ConvParams p) {
  pdl_wait();
  pdl_launch();
  int valid = p.d_valid ? min(*p.d_valid, p.rows) : p.valid;
  valid = max(valid, 0);
  const int cg8 = p.C >> 3;
  const int rows_per = (p.rows + gridDim.y - 1) / gridDim.y;
  const int c8 = blockIdx.x * blockDim.x + threadIdx.x;
  if (c8 >= cg8) return;
  const int b = blockIdx.z;
  const int r_lo = blockIdx.y * rows_per, r_hi = min(p.rows, r_lo + rows_per);
  const __nv_bfloat16* x = p.x + (size_t)b * p.x_batch + c8 * 8;
  const __nv_bfloat16* hist = p.history ? p.history + (size_t)b * p.hist_batch + c8 * 8 : nullptr;
  __nv_bfloat16* y = p.y + (size_t)b * p.y_batch + c8 * 8;

  const uint4 zero = make_uint4(0, 0, 0, 0);
  uint4 w[K], win[K], bias = zero;
#pragma unroll
  for (int k = 0; k < K; ++k) w[k] = ld_cached(p.taps + (size_t)k * p.C + c8 * 8);
  if (p.bias) bias = ld_cached(p.bias + c8 * 8);
  // row index r of the concatenation history ++ x is (r - (K-1)) of x
  auto input_row = [&](int r) -> uint4 {
    if (r >= 0) return r < valid ? ld_cached(x + (size_t)r * p.C) : zero;
    if (hist) return ld_cached(hist + (size_t)(r + K - 1) * p.C);
    return zero;
  };
#pragma unroll
  for (int k = 0; k < K - 1; ++k) win[k] = input_row(r_lo - (K - 1) + k);
  // Eight rows at a time: their loads are issued together, then the eight outputs follow.
  constexpr int kRows = 8;
  for (int r0 = r_lo; r0 < r_hi; r0 += kRows) {
    uint4 raw[kRows];
#pragma unroll
    for (int u = 0; u < kRows; ++u) {
      const int r = r0 + u;
      raw[u] = (r < r_hi && r < valid) ? ld_cached(x + (size_t)r * p.C) : zero;
    }
#pragma unroll
    for (int u = 0; u < kRows; ++u) {
      const int r = r0 + u;
      if (r >= r_hi) break;
      win[K - 1] = raw[u];
      uint4 out = zero;
      if (r < valid) {
        uint4 acc;
        if (p.decode_order) {
          acc = bmul8(win[K - 1], w[K - 1]);
#pragma unroll
          for (int k = 0; k < K - 1; ++k) acc = badd8(acc, bmul8(win[k], w[k]));
        } else {
          acc = bmul8(win[0], w[0]);
#pragma unroll
          for (int k = 1; k < K; ++k) acc = badd8(acc, bmul8(win[k], w[k]));
        }
        if (p.bias) acc = badd8(acc, bias);
        if (p.silu) {
          float f[8];
          unpack8(acc, f);
#pragma unroll
          for (int j = 0; j < 8; ++j) f[j] = silu_f32(f[j]);
          acc = pack8(f);
        }
        out = acc;
      }
      *reinterpret_cast<uint4*>(y + (size_t)r * p.C) = out;
#pragma unroll
      for (int k = 0; k < K - 1; ++k) win[k] = win[k + 1];
    }
  }
  // the K-1 rows ending the valid run become the next call's history
  if (p.new_history && blockIdx.y == 0) {
    __nv_bfloat16* nh = p.new_history + (size_t)b * p.hist_batch + c8 * 8;
    uint4 keep[K - 1];
#pragma unroll
    for (int k = 0; k < K - 1; ++k) keep[k] = input_row(valid - (K - 1) + k);
#pragma unroll
    for (int k = 0; k < K - 1; ++k) *reinterpret_cast<uint4*>(nh + (size_t)k * p.C) = keep[k];
  }
}


// ---------------------------------------------------------------- chunked scan (tensor cores)
// The same recurrence in the chunked ("state-space dual") form for prompt-length calls.  With
// a_t = step_t * A (<= 0) and cum_t the running sum of a over a chunk of Q = 64 rows,
//
//   y_t     = sum_{j <= t} exp(cum_t - cum_j) step_j (C_t . B_j) x_j  +  exp(cum_t) C_t . S_prev  +  D x_t
//   S_next  = exp(cum_Q) S_prev  +  sum_j exp(cum_Q - cum_j) step_j  x_j (x) B_j
//
// so a chunk is four small matrix products instead of 64 dependent steps: the scores
// C B^T (Q x Q over the state axis), the decay-masked scores times X (Q x P), C times the
// carried state (Q x P over the state axis) and the state update X_w^T B (P x N over the
// chunk's rows).  All four run as bf16 mma.sync with float32 accumulation: x, B and C are
// the call's own bf16 inputs (exact), the decay-masked scores, the weighted rows x_j w_j and
// the carried state are rounded to bf16 once each as operands.  The decays are differences
// of the float32 running sum (never a product of 64 factors) and every difference is <= 0,
// so nothing overflows.  The state itself stays in float32 registers from chunk to chunk.
// One CTA of four warps owns one (sequence, head): warp w owns rows 16 w .. 16 w + 15 of
// every Q-row tile and rows 16 w .. of the (P x N) state; three CTAs share an SM, which is
// what overlaps one CTA's loads with its neighbours' products.
constexpr int kSsdQ = 64;       // rows per chunk
constexpr int kSsdP = 64;       // head_dim this kernel takes
constexpr int kSsdThreads = 128;

template <int N>
struct SsdSmem {
  static constexpr int PX = kSsdP + 8, PN = N + 8;                   // row pitches in elements
  static constexpr size_t off_x = 0;
  static constexpr size_t off_b = off_x + (size_t)kSsdQ * PX * 2;
  static constexpr size_t off_c = off_b + (size_t)kSsdQ * PN * 2;
  static constexpr int PZ = kSsdP + 4;                              // floats
  static constexpr size_t off_z = off_c + (size_t)kSsdQ * PN * 2;    // C S_prev^T, float32; then a warp's rows of y
  static constexpr size_t off_f = off_z + (size_t)kSsdQ * PZ * 4;    // cum, step, w, exp(cum): 4 x Q floats
  static constexpr size_t total = off_f + 4 * kSsdQ * sizeof(float);
};

#ifndef SSD_DROP
#define SSD_DROP 0   // bit 0: masked scores, bit 1: weighted rows, bit 2: state -- as one bf16 operand only
#endif

template <int N>
__global__ void __launch_bounds__(kSsdThreads, 3) ssd_scan_kernel(const ScanParams p) {
  using S = SsdSmem<N>;
  constexpr int Q = kSsdQ, P = kSsdP, PX = S::PX, PN = S::PN, PZ = S::PZ;
  extern __shared__ __align__(128) unsigned char ssd_smem[];
  __nv_bfloat16* sX = reinterpret_cast<__nv_bfloat16*>(ssd_smem + S::off_x);
  __nv_bfloat16* sB = reinterpret_cast<__nv_bfloat16*>(ssd_smem + S::off_b);
  __nv_bfloat16* sC = reinterpret_cast<__nv_bfloat16*>(ssd_smem + S::off_c);
  float* sZ = reinterpret_cast<float*>(ssd_smem + S::off_z);
  float* s_cum = reinterpret_cast<float*>(ssd_smem + S::off_f);
  float* s_step = s_cum + Q;
  float* s_w = s_step + Q;
  float* s_ecum = s_w + Q;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g4 = lane >> 2, t4 = lane & 3;
  const int h = blockIdx.x, b = blockIdx.y;
  const int grp = h / (p.H / p.G);
  const int inner = p.H * P;
  pdl_wait();
  pdl_launch();
  int valid = p.d_valid ? min(*p.d_valid, p.rows) : p.valid;
  valid = max(valid, 0);
  const float dt_bias = p.head[h * 3], A = p.head[h * 3 + 1], Dh = p.head[h * 3 + 2];
  const __nv_bfloat16* xbc = p.xbc + (size_t)b * p.xbc_batch;
  const __nv_bfloat16* dtp = p.dt + (size_t)b * p.dt_batch;
  __nv_bfloat16* yb = p.y + (size_t)b * p.y_batch;

  // the state: warp w holds rows 16 w + g4 and + 8, columns 8 i + 2 t4, + 1 of every n-tile i
  float st[N / 8][4];
  {
    const float* src = p.state ? p.state + (size_t)b * p.state_batch + (size_t)h * P * N : nullptr;
#pragma unroll
    for (int i = 0; i < N / 8; ++i) {
      const int r0 = 16 * warp + g4, n0 = 8 * i + 2 * t4;
      float2 lo = make_float2(0.f, 0.f), hi = lo;
      if (src) {
        lo = *reinterpret_cast<const float2*>(src + (size_t)r0 * N + n0);
        hi = *reinterpret_cast<const float2*>(src + (size_t)(r0 + 8) * N + n0);
      }
      st[i][0] = lo.x; st[i][1] = lo.y; st[i][2] = hi.x; st[i][3] = hi.y;
    }
  }

  auto cp16 = [](void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
  };
  auto load_rows = [&](__nv_bfloat16* dst, int pitch, int width16, size_t col0, int c0) {
    // rows c0 .. c0 + Q - 1 of the call, `width16` 16-byte pieces from column col0; rows past the call are zeros
    for (int idx = tid; idx < Q * width16; idx += kSsdThreads) {
      const int r = idx / width16, ch = idx - r * width16;
      __nv_bfloat16* d = dst + (size_t)r * pitch + ch * 8;
      if (c0 + r < p.rows) cp16(d, xbc + (size_t)(c0 + r) * p.width + col0 + ch * 8);
      else *reinterpret_cast<uint4*>(d) = make_uint4(0, 0, 0, 0);
    }
  };
  // a float32 pair as a bf16 head and the bf16 of what the head left over
  auto split = [](float v0, float v1, uint32_t& hi, uint32_t& lo) {
    hi = pack_bf16x2(v0, v1);
    lo = pack_bf16x2(v0 - bf16_lo(hi), v1 - bf16_hi(hi));
  };

  const int r_lo = 16 * warp + g4, r_hi = r_lo + 8;        // this lane's two rows of every 16-row tile
  for (int c0 = 0; c0 < p.rows; c0 += Q) {
    // ---- the chunk's rows of x, B and C; meanwhile warp 0 turns the chunk's steps into their
    // running sum (lane l: rows l and l + 32) and the decays every product below needs ----
    load_rows(sX, PX, P / 8, (size_t)h * P, c0);
    load_rows(sB, PN, N / 8, (size_t)inner + (size_t)grp * N, c0);
    load_rows(sC, PN, N / 8, (size_t)inner + (size_t)(p.G + grp) * N, c0);
    if (warp == 0) {
      float step[2], cum[2];
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int t = c0 + lane + 32 * u;
        step[u] = t < valid ? softplus_f32(__bfloat162float(dtp[(size_t)t * p.H + h]) + dt_bias) : 0.f;
        float a = step[u] * A;                             // rows past the bound: a = 0, step = 0
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
          const float v = __shfl_up_sync(0xffffffffu, a, off);
          if (lane >= off) a += v;
        }
        cum[u] = a;
      }
      cum[1] += __shfl_sync(0xffffffffu, cum[0], 31);     // the first half's total carries into the second
      const float total = __shfl_sync(0xffffffffu, cum[1], 31);
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int r = lane + 32 * u;
        s_cum[r] = cum[u];
        s_step[r] = step[u];
        s_ecum[r] = __expf(cum[u]);
        s_w[r] = __expf(total - cum[u]) * step[u];
      }
    }
    asm volatile("cp.async.commit_group;\n\tcp.async.wait_group 0;" ::: "memory");
    __syncthreads();

    // ---- Z = C S_prev^T for all rows of the chunk and this warp's 16 columns: the carried
    // state is the B operand straight from the registers that hold it (the accumulator layout
    // of two 8-column tiles is the B-fragment layout of a 16-deep step), split into a bf16
    // head and remainder so that the read-out keeps float32's accuracy.  Products that add
    // into the same accumulator are issued as far apart as the registers allow ----
    {
      float zt[Q / 16][2][4];
#pragma unroll
      for (int mt = 0; mt < Q / 16; ++mt)
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) { zt[mt][nt][0] = zt[mt][nt][1] = zt[mt][nt][2] = zt[mt][nt][3] = 0.f; }
#pragma unroll
      for (int ks = 0; ks < N / 16; ++ks) {
        uint32_t bh[2][2], bl[2][2];     // [column tile: rows r_lo / r_hi of the state][k half]
#pragma unroll
        for (int kh = 0; kh < 2; ++kh) {
          const float* v = st[2 * ks + kh];
          split(v[0], v[1], bh[0][kh], bl[0][kh]);
          split(v[2], v[3], bh[1][kh], bl[1][kh]);
        }
#pragma unroll
        for (int mp = 0; mp < Q / 32; ++mp) {
          uint32_t a0[4], a1[4];
          load_a_rowmajor(a0, sC, PN, 32 * mp, ks * 16, lane);
          load_a_rowmajor(a1, sC, PN, 32 * mp + 16, ks * 16, lane);
          mma_bf16_16816(zt[2 * mp][0], a0, bh[0][0], bh[0][1]);
          mma_bf16_16816(zt[2 * mp][1], a0, bh[1][0], bh[1][1]);
          mma_bf16_16816(zt[2 * mp + 1][0], a1, bh[0][0], bh[0][1]);
          mma_bf16_16816(zt[2 * mp + 1][1], a1, bh[1][0], bh[1][1]);
          if (!(SSD_DROP & 4)) {
            mma_bf16_16816(zt[2 * mp][0], a0, bl[0][0], bl[0][1]);
            mma_bf16_16816(zt[2 * mp][1], a0, bl[1][0], bl[1][1]);
            mma_bf16_16816(zt[2 * mp + 1][0], a1, bl[0][0], bl[0][1]);
            mma_bf16_16816(zt[2 * mp + 1][1], a1, bl[1][0], bl[1][1]);
          }
        }
      }
#pragma unroll
      for (int mt = 0; mt < Q / 16; ++mt)
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
          const int col = 16 * warp + 8 * nt + 2 * t4;
          *reinterpret_cast<float2*>(sZ + (size_t)(16 * mt + g4) * PZ + col) = make_float2(zt[mt][nt][0], zt[mt][nt][1]);
          *reinterpret_cast<float2*>(sZ + (size_t)(16 * mt + g4 + 8) * PZ + col) = make_float2(zt[mt][nt][2], zt[mt][nt][3]);
        }
    }

    // ---- scores S = C B^T, masked and decayed into M (rows of this warp) ----
    uint32_t m_hi[Q / 16][4], m_lo[Q / 16][4];
    {
      float acc[Q / 8][4];
#pragma unroll
      for (int i = 0; i < Q / 8; ++i) { acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f; }
#pragma unroll
      for (int ks = 0; ks < N / 16; ++ks) {
        uint32_t a[4];
        load_a_rowmajor(a, sC, PN, 16 * warp, ks * 16, lane);
#pragma unroll
        for (int i2 = 0; i2 < Q / 16; ++i2) {
          uint32_t bb[4];
          load_b_nk(bb, sB, PN, i2 * 16, ks * 16, lane);
          mma_bf16_16816(acc[2 * i2], a, bb[0], bb[1]);
          mma_bf16_16816(acc[2 * i2 + 1], a, bb[2], bb[3]);
        }
      }
      // The accumulator layout of two adjacent 8-column tiles is the A-fragment layout of one
      // 16-deep step, so the masked scores go straight back into the tensor cores from
      // registers, split into a bf16 head and a bf16 remainder (two products) to keep float32's
      // accuracy.
      const float cl = s_cum[r_lo], ch = s_cum[r_hi];
#pragma unroll
      for (int i = 0; i < Q / 8; ++i) {
        const int j0 = 8 * i + 2 * t4, j1 = j0 + 1;
        const float2 cj = *reinterpret_cast<const float2*>(s_cum + j0);
        const float2 sj = *reinterpret_cast<const float2*>(s_step + j0);
        const float m00 = j0 <= r_lo ? acc[i][0] * __expf(cl - cj.x) * sj.x : 0.f;
        const float m01 = j1 <= r_lo ? acc[i][1] * __expf(cl - cj.y) * sj.y : 0.f;
        const float m10 = j0 <= r_hi ? acc[i][2] * __expf(ch - cj.x) * sj.x : 0.f;
        const float m11 = j1 <= r_hi ? acc[i][3] * __expf(ch - cj.y) * sj.y : 0.f;
        const int ks = i >> 1, half = (i & 1) * 2;        // tile i is k-columns 8 (i & 1) .. of step i / 2
        split(m00, m01, m_hi[ks][half], m_lo[ks][half]);
        split(m10, m11, m_hi[ks][half + 1], m_lo[ks][half + 1]);
      }
    }
    __syncthreads();   // Z is whole

    // ---- y = M X  +  exp(cum_t) Z  +  D x  (rows of this warp) ----
    {
      float y[P / 8][4];
#pragma unroll
      for (int i = 0; i < P / 8; ++i) { y[i][0] = y[i][1] = y[i][2] = y[i][3] = 0.f; }
#pragma unroll
      for (int ks = 0; ks < Q / 16; ++ks) {
#pragma unroll
        for (int ip = 0; ip < P / 32; ++ip) {
          uint32_t b0[4], b1[4];
          load_b_kn(b0, sX, PX, ip * 32, ks * 16, lane);
          load_b_kn(b1, sX, PX, ip * 32 + 16, ks * 16, lane);
          mma_bf16_16816(y[4 * ip], m_hi[ks], b0[0], b0[1]);
          mma_bf16_16816(y[4 * ip + 1], m_hi[ks], b0[2], b0[3]);
          mma_bf16_16816(y[4 * ip + 2], m_hi[ks], b1[0], b1[1]);
          mma_bf16_16816(y[4 * ip + 3], m_hi[ks], b1[2], b1[3]);
          if (!(SSD_DROP & 1)) {
            mma_bf16_16816(y[4 * ip], m_lo[ks], b0[0], b0[1]);
            mma_bf16_16816(y[4 * ip + 1], m_lo[ks], b0[2], b0[3]);
            mma_bf16_16816(y[4 * ip + 2], m_lo[ks], b1[0], b1[1]);
            mma_bf16_16816(y[4 * ip + 3], m_lo[ks], b1[2], b1[3]);
          }
        }
      }
      const float el = s_ecum[r_lo], eh = s_ecum[r_hi];
      const bool live_lo = c0 + r_lo < valid, live_hi = c0 + r_hi < valid;
      uint32_t out_lo[P / 8], out_hi[P / 8];
#pragma unroll
      for (int i = 0; i < P / 8; ++i) {
        const int p0 = 8 * i + 2 * t4;
        const uint32_t xl = *reinterpret_cast<const uint32_t*>(sX + (size_t)r_lo * PX + p0);
        const uint32_t xh = *reinterpret_cast<const uint32_t*>(sX + (size_t)r_hi * PX + p0);
        const float2 zl = *reinterpret_cast<const float2*>(sZ + (size_t)r_lo * PZ + p0);
        const float2 zh = *reinterpret_cast<const float2*>(sZ + (size_t)r_hi * PZ + p0);
        const float v00 = fmaf(Dh, bf16_lo(xl), fmaf(el, zl.x, y[i][0]));
        const float v01 = fmaf(Dh, bf16_hi(xl), fmaf(el, zl.y, y[i][1]));
        const float v10 = fmaf(Dh, bf16_lo(xh), fmaf(eh, zh.x, y[i][2]));
        const float v11 = fmaf(Dh, bf16_hi(xh), fmaf(eh, zh.y, y[i][3]));
        out_lo[i] = live_lo ? pack_bf16x2(v00, v01) : 0u;
        out_hi[i] = live_hi ? pack_bf16x2(v10, v11) : 0u;
      }
      // The warp's 16 rows of y are staged over its own rows of Z (which only it reads, and has
      // read) and leave as 128-byte rows.
      __syncwarp();
      __nv_bfloat16* stage = reinterpret_cast<__nv_bfloat16*>(sZ);
      constexpr int PS = PZ * 2;                           // the same row pitch, in bf16 elements
#pragma unroll
      for (int i = 0; i < P / 8; ++i) {
        const int p0 = 8 * i + 2 * t4;
        *reinterpret_cast<uint32_t*>(stage + (size_t)r_lo * PS + p0) = out_lo[i];
        *reinterpret_cast<uint32_t*>(stage + (size_t)r_hi * PS + p0) = out_hi[i];
      }
      __syncwarp();
      for (int idx = lane; idx < 16 * (P / 8); idx += 32) {
        const int r = idx / (P / 8), ch = idx - r * (P / 8);
        const int t = c0 + 16 * warp + r;
        if (t < p.rows)
          *reinterpret_cast<uint4*>(yb + (size_t)t * inner + (size_t)h * P + ch * 8) =
              *reinterpret_cast<const uint4*>(stage + (size_t)(16 * warp + r) * PS + ch * 8);
      }
    }

    // ---- S = exp(cum_Q) S + X_w^T B.  The weighted rows x_j w_j are made in registers from
    // the transposed fragments of x (a register holds rows j, j + 1 of one column), rounded to
    // bf16 as an operand, their remainders going through a second product, so the state keeps
    // float32's accuracy from chunk to chunk ----
    {
      const float decay = s_ecum[Q - 1];
#pragma unroll
      for (int i = 0; i < N / 8; ++i) { st[i][0] *= decay; st[i][1] *= decay; st[i][2] *= decay; st[i][3] *= decay; }
#pragma unroll
      for (int ks = 0; ks < Q / 16; ++ks) {
        uint32_t raw[4], a[4], al[4];
        load_a_transposed(raw, sX, PX, 16 * warp, ks * 16, lane);
        const float2 w0 = *reinterpret_cast<const float2*>(s_w + ks * 16 + 2 * t4);
        const float2 w1 = *reinterpret_cast<const float2*>(s_w + ks * 16 + 8 + 2 * t4);
        split(bf16_lo(raw[0]) * w0.x, bf16_hi(raw[0]) * w0.y, a[0], al[0]);
        split(bf16_lo(raw[1]) * w0.x, bf16_hi(raw[1]) * w0.y, a[1], al[1]);
        split(bf16_lo(raw[2]) * w1.x, bf16_hi(raw[2]) * w1.y, a[2], al[2]);
        split(bf16_lo(raw[3]) * w1.x, bf16_hi(raw[3]) * w1.y, a[3], al[3]);
#pragma unroll
        for (int ip = 0; ip < N / 32; ++ip) {
          uint32_t b0[4], b1[4];
          load_b_kn(b0, sB, PN, ip * 32, ks * 16, lane);
          load_b_kn(b1, sB, PN, ip * 32 + 16, ks * 16, lane);
          mma_bf16_16816(st[4 * ip], a, b0[0], b0[1]);
          mma_bf16_16816(st[4 * ip + 1], a, b0[2], b0[3]);
          mma_bf16_16816(st[4 * ip + 2], a, b1[0], b1[1]);
          mma_bf16_16816(st[4 * ip + 3], a, b1[2], b1[3]);
          if (!(SSD_DROP & 2)) {
            mma_bf16_16816(st[4 * ip], al, b0[0], b0[1]);
            mma_bf16_16816(st[4 * ip + 1], al, b0[2], b0[3]);
            mma_bf16_16816(st[4 * ip + 2], al, b1[0], b1[1]);
            mma_bf16_16816(st[4 * ip + 3], al, b1[2], b1[3]);
          }
        }
      }
    }
    __syncthreads();   // x, B, C, Z and the decays are free for the next chunk
  }

  if (p.final_state) {
    float* dst = p.final_state + (size_t)b * p.state_batch + (size_t)h * P * N;
    const int r0 = 16 * warp + g4;
#pragma unroll
    for (int i = 0; i < N / 8; ++i) {
      const int n0 = 8 * i + 2 * t4;
      *reinterpret_cast<float2*>(dst + (size_t)r0 * N + n0) = make_float2(st[i][0], st[i][1]);
      *reinterpret_cast<float2*>(dst + (size_t)(r0 + 8) * N + n0) = make_float2(st[i][2], st[i][3]);
    }
  }
}

template <int N>
static int launch_ssd(const ScanParams& p, int batch, cudaStream_t stream) {
  static DeviceOnce configured;   // the attribute is per device
  if (!configured.done()) {
    if (cudaFuncSetAttribute(ssd_scan_kernel<N>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)SsdSmem<N>::total) != cudaSuccess)
      return IRON_ERR_LAUNCH;
    configured.mark();
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(p.H, batch);
  cfg.blockDim = dim3(kSsdThreads);
  cfg.dynamicSmemBytes = SsdSmem<N>::total;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  fill_pdl_attr(cfg, attr);
  return cudaLaunchKernelEx(&cfg, ssd_scan_kernel<N>, p) == cudaSuccess ? IRON_OK : IRON_ERR_LAUNCH;
}

// Calls of a prompt's length on the shapes the chunked kernels take run on them: 2 (the default)
// = the tcgen05 kernel where its shape fits (64-wide heads, 128 states, 128 rows or more), else
// the warp-MMA kernel; 1 = the warp-MMA kernel only; 0 (IRON_SCAN_CHUNKED=0) keeps every call on
// the step-by-step kernel.
static std::atomic<int> g_ssd_on{-1};
static int ssd_mode() {
  int on = g_ssd_on.load(std::memory_order_relaxed);
  if (on < 0) {
    const char* e = getenv("IRON_SCAN_CHUNKED");
    on = (e && e[0] >= '0' && e[0] <= '2') ? e[0] - '0' : 2;
    g_ssd_on.store(on, std::memory_order_relaxed);
  }
  return on;
}
static bool ssd_enabled() { return ssd_mode() != 0; }
static int* g_scan_status[64] = {};   // one status word per device

template <typename... Args>
static int launch_scan_pdl(void (*kernel)(Args...), dim3 grid, dim3 block, cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  fill_pdl_attr(cfg, attr);
  return cudaLaunchKernelEx(&cfg, kernel, args...) == cudaSuccess ? IRON_OK : IRON_ERR_LAUNCH;
}

}  // namespace iron

using namespace iron;

extern "C" void iron_set_scan_chunked(int mode) {
  g_ssd_on.store(mode < 0 ? 0 : (mode > 2 ? 2 : mode), std::memory_order_relaxed);
}
extern "C" void iron_selective_scan_status_word(int* d_status) {
  const int dev = current_device();
  if (dev >= 0) g_scan_status[dev] = d_status;
}

extern "C" int iron_selective_scan_bf16(const void* xbc, const void* dt, const void* head, const void* state,
                                        void* y, void* final_state, int batch, int rows, int heads,
                                        int head_dim, int state_size, int groups, int valid_rows,
                                        const int* d_valid_rows, iron_stream_t stream) {
  if (batch <= 0 || rows <= 0 || heads <= 0 || groups <= 0 || heads % groups) return IRON_ERR_SHAPE;
  if (head_dim <= 0 || (head_dim & 7)) return IRON_ERR_SHAPE;
  if (state_size != 16 && state_size != 32 && state_size != 64 && state_size != 128) return IRON_ERR_SHAPE;
  if (valid_rows < 0 || valid_rows > rows) return IRON_ERR_SHAPE;
  if (!aligned16(xbc) || !aligned16(y) || !aligned16(head)) return IRON_ERR_ALIGN;
  if ((state && !aligned16(state)) || (final_state && !aligned16(final_state))) return IRON_ERR_ALIGN;
  ScanParams p = {};
  p.xbc = (const __nv_bfloat16*)xbc; p.dt = (const __nv_bfloat16*)dt; p.head = (const float*)head;
  p.state = (const float*)state; p.y = (__nv_bfloat16*)y; p.final_state = (float*)final_state;
  p.rows = rows; p.H = heads; p.P = head_dim; p.G = groups;
  p.width = heads * head_dim + 2 * groups * state_size;
  if (p.width & 7) return IRON_ERR_SHAPE;
  p.valid = valid_rows; p.d_valid = d_valid_rows;
  p.xbc_batch = (long long)rows * p.width; p.dt_batch = (long long)rows * heads;
  p.y_batch = (long long)rows * heads * head_dim;
  p.state_batch = (long long)heads * head_dim * state_size;
  // Four threads per row pair (64 rows per CTA); eight, with twice the CTAs, measured slower
  // at 48 heads x 64 x 128 (3.4 ms against 2.3 ms): the staging of B and C doubles.
  const dim3 block(kScanThreads);
  const dim3 grid64(heads * ((head_dim + 63) / 64), batch);
  cudaStream_t s = (cudaStream_t)stream;
  if (head_dim == kSsdP && state_size == 128 && rows >= 128 && ssd_mode() == 2) {   // tcgen05, 128-row chunks
    const int dev = current_device();
    const int rc = launch_ssd_tc(p, batch, s, dev >= 0 ? g_scan_status[dev] : nullptr);
    if (rc != IRON_ERR_UNSUPPORTED) return rc;
  }
  if (head_dim == kSsdP && rows >= 32 && ssd_enabled()) {   // the chunked form on warp MMAs
    if (state_size == 128) return launch_ssd<128>(p, batch, s);
    if (state_size == 64) return launch_ssd<64>(p, batch, s);
  }
  switch (state_size) {
    case 16: return launch_scan_pdl(selective_scan_kernel<16, 4>, grid64, block, s, p);
    case 32: return launch_scan_pdl(selective_scan_kernel<32, 4>, grid64, block, s, p);
    case 64: return launch_scan_pdl(selective_scan_kernel<64, 4>, grid64, block, s, p);
    default: return launch_scan_pdl(selective_scan_kernel<128, 4>, grid64, block, s, p);
  }
}

extern "C" int iron_causal_conv1d_bf16(const void* x, const void* taps, const void* bias, const void* history,
                                       void* new_history, void* y, int batch, int rows, int channels,
                                       int kernel, int valid_rows, const int* d_valid_rows, int decode_order,
                                       int silu, iron_stream_t stream) {
  if (batch <= 0 || rows <= 0 || channels <= 0 || (channels & 7)) return IRON_ERR_SHAPE;
  if (kernel < 2 || kernel > 4) return IRON_ERR_SHAPE;
  if (valid_rows < 0 || valid_rows > rows) return IRON_ERR_SHAPE;
  if (!aligned16(x) || !aligned16(taps) || !aligned16(y)) return IRON_ERR_ALIGN;
  if ((bias && !aligned16(bias)) || (history && !aligned16(history)) || (new_history && !aligned16(new_history)))
    return IRON_ERR_ALIGN;
  ConvParams p = {};
  p.x = (const __nv_bfloat16*)x; p.taps = (const __nv_bfloat16*)taps; p.bias = (const __nv_bfloat16*)bias;
  p.history = (const __nv_bfloat16*)history; p.new_history = (__nv_bfloat16*)new_history;
  p.y = (__nv_bfloat16*)y;
  p.rows = rows; p.C = channels; p.K = kernel; p.valid = valid_rows; p.d_valid = d_valid_rows;
  p.decode_order = decode_order; p.silu = silu;
  p.x_batch = p.y_batch = (long long)rows * channels;
  p.hist_batch = (long long)(kernel - 1) * channels;
  // rows are cut into segments so a long prompt fills the machine; each segment re-reads
  // the K-1 rows before it
  // a thread takes 8 channels; the block is the multiple of 32 threads (up to 128) that wastes the fewest
  // lanes on the last block of a row (3328 channels = 416 threads' worth: 13 blocks of 32, none idle)
  const int c8s = channels / 8;
  int threads = 128, idle = (128 - c8s % 128) % 128;
  for (int t = 96; t >= 32; t -= 32) {
    const int waste = (t - c8s % t) % t;
    if (waste < idle) { threads = t; idle = waste; }
  }
  const int cgroups = (c8s + threads - 1) / threads;
  int segs = (16 * kSMs * (128 / threads) + cgroups * batch - 1) / (cgroups * batch);
  segs = segs < 1 ? 1 : segs;
  const int max_segs = (rows + 31) / 32;
  if (segs > max_segs) segs = max_segs;
  const dim3 grid(cgroups, segs, batch), block(threads);
  cudaStream_t s = (cudaStream_t)stream;
  switch (kernel) {
    case 2: return launch_scan_pdl(causal_conv_kernel<2>, grid, block, s, p);
    case 3: return launch_scan_pdl(causal_conv_kernel<3>, grid, block, s, p);
    default: return launch_scan_pdl(causal_conv_kernel<4>, grid, block, s, p);
  }
}
