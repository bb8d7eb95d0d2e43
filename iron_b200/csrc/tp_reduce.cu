// All-reduce of a small bf16 vector over the tensor-parallel ranks through peer memory,
// fused with the residual add that follows it in a decoder layer.
//
// At batch 1 the row-parallel projections (o_proj, down_proj) leave each rank a partial
// sum of a few kilobytes, 56 times per token.  A library all-reduce costs ~15 us of launch
// and protocol latency each; here one small kernel per rank
//   1. stores its partial into slot [parity][rank] of EVERY rank's buffer (plain stores to
//      peer memory over NVLink) and then, after a system-scope fence, raises that slot's
//      flag on every rank to the sequence number of this all-reduce;
//   2. waits (bounded) until the flags of all ranks in its own buffer carry that number;
//   3. adds the partials in rank order in f32, rounds once to bf16, adds the residual and
//      rounds again -- the same value on every rank.
// The buffers are double-buffered by the parity of the sequence number: a rank can be at
// most one all-reduce ahead of its slowest peer, because it cannot pass step 2 of the next
// one without that peer's flag.  Flags only ever grow, so nothing is reset.
//
// The wait is bounded by a wall-clock limit; a rank that gives up records IRON_ERR_TIMEOUT
// in the status word and finishes with whatever it has, so a missing peer never hangs the
// GPU.  No multicast and no multimem: plain loads and stores.
#include "common.cuh"

namespace iron {

constexpr int kTpMaxWorld = 8;
constexpr int kTpFlagBytes = 256;                      // flags sit ahead of the slots
constexpr unsigned long long kTpWaitNs = 2000000000ull;  // 2 s

struct TpParams {
  const __nv_bfloat16* part;      // this rank's partial (n)
  const __nv_bfloat16* residual;  // optional (n)
  __nv_bfloat16* y;               // (n)
  int n, slot_elems, rank, world;
  unsigned char* peer[kTpMaxWorld];  // every rank's buffer: flags, then slots [2][world][slot_elems]
  unsigned int* d_seq;            // this rank's sequence counter
  int* status;
};

__device__ __forceinline__ unsigned int tp_ld_acquire_sys(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void tp_st_release_sys(unsigned int* p, unsigned int v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned long long tp_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

__global__ void __launch_bounds__(512) tp_allreduce_kernel(const TpParams p) {
  pdl_wait();
  pdl_launch();
  const int tid = threadIdx.x;
  const unsigned int seq = *p.d_seq;
  const unsigned int par = seq & 1u;
  const int n8 = p.n >> 3;
  const size_t slot16 = (size_t)p.slot_elems >> 3;   // uint4 per slot
  // 1. my partial into slot [par][rank] of every rank
  for (int i = tid; i < n8; i += blockDim.x) {
    const uint4 v = ld_cached(reinterpret_cast<const uint4*>(p.part) + i);
    for (int r = 0; r < p.world; ++r) {
      uint4* slots = reinterpret_cast<uint4*>(p.peer[r] + kTpFlagBytes);
      slots[((size_t)par * p.world + p.rank) * slot16 + i] = v;
    }
  }
  __threadfence_system();
  __syncthreads();
  if (tid < p.world)
    tp_st_release_sys(reinterpret_cast<unsigned int*>(p.peer[tid]) + par * p.world + p.rank, seq + 1u);
  // 2. everyone's partial is in my buffer
  if (tid < p.world) {
    const unsigned int* flag = reinterpret_cast<const unsigned int*>(p.peer[p.rank]) + par * p.world + tid;
    if ((int)(tp_ld_acquire_sys(flag) - (seq + 1u)) < 0) {
      const unsigned long long t0 = tp_ns();
      for (unsigned int it = 1;; ++it) {
        if ((int)(tp_ld_acquire_sys(flag) - (seq + 1u)) >= 0) break;
        if ((it & 63u) == 0 && tp_ns() - t0 > kTpWaitNs) {
          if (p.status) *reinterpret_cast<volatile int*>(p.status) = IRON_ERR_TIMEOUT;
          break;
        }
      }
    }
  }
  __syncthreads();
  // 3. sum in rank order, round, add the residual, round
  const uint4* mine = reinterpret_cast<const uint4*>(p.peer[p.rank] + kTpFlagBytes) + (size_t)par * p.world * slot16;
  for (int i = tid; i < n8; i += blockDim.x) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int r = 0; r < p.world; ++r) {
      float f[8];
      unpack8(__ldcv(mine + (size_t)r * slot16 + i), f);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += f[j];
    }
    if (p.residual) {
      float f[8];
      unpack8(ld_cached(reinterpret_cast<const uint4*>(p.residual) + i), f);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = __fadd_rn(round_bf16(acc[j]), f[j]);
    }
    reinterpret_cast<uint4*>(p.y)[i] = pack8(acc);
  }
  if (tid == 0) *p.d_seq = seq + 1u;
}

// ---------------------------------------------------------------------------------------------
// The same all-reduce without a fence or a flag, for a few rows (a decode batch): every value
// travels as one 32-bit word -- the bf16 partial and a 16-bit tag of the exchange's number -- and a
// word arrives whole, so its tag says that its value is there.  Many CTAs, each taking a run of
// the elements: store the words into slot [parity][rank] of every rank, then read every rank's
// words of that run from the own buffer, again while a tag is not yet this exchange's (at most 2 s).
// The last CTA to finish advances the rank's exchange number.  Slots and tags are those of the
// exchange folded into the GEMVs (gemv.cu); an engine uses one of the three forms on a buffer.
struct TpTaggedParams {
  const __nv_bfloat16* part;
  const __nv_bfloat16* residual;
  __nv_bfloat16* y;
  int n, slot_elems, rank, world;
  unsigned char* peer[kTpMaxWorld];
  unsigned int* state;            // [0] exchange number, [1] CTAs that have finished this launch
  int* status;
};

__global__ void __launch_bounds__(256) tp_allreduce_tagged_kernel(const TpTaggedParams p) {
  pdl_wait();
  pdl_launch();
  const unsigned int seq = p.state[0], par = seq & 1u, tag = ((seq >> 1) + 1u) & 0xffffu;
  const int n4 = p.n >> 2;
  const size_t base = ((size_t)par * p.world) * p.slot_elems;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += gridDim.x * blockDim.x) {
    // 1. four partials as tagged words into slot [par][rank] of every rank
    const uint2 raw = *reinterpret_cast<const uint2*>(p.part + 4 * (size_t)i);
    const uint32_t t = tag << 16;
    const uint4 words = make_uint4((raw.x & 0xffffu) | t, (raw.x >> 16) | t, (raw.y & 0xffffu) | t, (raw.y >> 16) | t);
    for (int r = 0; r < p.world; ++r) {
      uint32_t* dst = reinterpret_cast<uint32_t*>(p.peer[r] + kTpFlagBytes) + base + (size_t)p.rank * p.slot_elems + 4 * (size_t)i;
      asm volatile("st.relaxed.sys.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "r"(words.x), "r"(words.y),
                   "r"(words.z), "r"(words.w) : "memory");
    }
  }
  bool gave_up = false;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += gridDim.x * blockDim.x) {
    // 2. every rank's four words from the own buffer, in rank order
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (int r = 0; r < p.world; ++r) {
      const uint32_t* src = reinterpret_cast<const uint32_t*>(p.peer[p.rank] + kTpFlagBytes) + base + (size_t)r * p.slot_elems + 4 * (size_t)i;
      uint4 w;
      unsigned long long t0 = 0;
      for (unsigned int it = 1;; ++it) {
        asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(w.x), "=r"(w.y), "=r"(w.z), "=r"(w.w) : "l"(src) : "memory");
        if ((w.x >> 16) == tag && (w.y >> 16) == tag && (w.z >> 16) == tag && (w.w >> 16) == tag) break;
        if (gave_up) break;
        if ((it & 63u) == 0) {
          const unsigned long long now = tp_ns();
          if (t0 == 0) t0 = now;
          else if (now - t0 > kTpWaitNs) { gave_up = true; break; }
        }
      }
      // a word that never came counts as zero
      acc[0] += (w.x >> 16) == tag ? __uint_as_float(w.x << 16) : 0.f;
      acc[1] += (w.y >> 16) == tag ? __uint_as_float(w.y << 16) : 0.f;
      acc[2] += (w.z >> 16) == tag ? __uint_as_float(w.z << 16) : 0.f;
      acc[3] += (w.w >> 16) == tag ? __uint_as_float(w.w << 16) : 0.f;
    }
    if (p.residual) {
      const uint2 rr = *reinterpret_cast<const uint2*>(p.residual + 4 * (size_t)i);
      acc[0] = __fadd_rn(round_bf16(acc[0]), bf16_lo(rr.x)); acc[1] = __fadd_rn(round_bf16(acc[1]), bf16_hi(rr.x));
      acc[2] = __fadd_rn(round_bf16(acc[2]), bf16_lo(rr.y)); acc[3] = __fadd_rn(round_bf16(acc[3]), bf16_hi(rr.y));
    }
    *reinterpret_cast<uint2*>(p.y + 4 * (size_t)i) = make_uint2(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]));
  }
  if (gave_up && p.status) *reinterpret_cast<volatile int*>(p.status) = IRON_ERR_TIMEOUT;
  // 3. the last CTA advances the exchange number (the next launch reads it after this one has ended)
  __syncthreads();
  if (threadIdx.x == 0) {
    if (atomicAdd(&p.state[1], 1u) == gridDim.x - 1) {
      p.state[1] = 0;
      p.state[0] = seq + 1u;
    }
  }
}

}  // namespace iron

using namespace iron;

extern "C" size_t iron_tp_buffer_bytes(int world, int slot_elems) {
  if (world <= 0 || world > kTpMaxWorld || slot_elems <= 0) return 0;
  // room for the tagged 32-bit words of an exchange folded into the GEMVs (gemv.cu); this kernel's bf16
  // slots take the first half
  return kTpFlagBytes + (size_t)2 * world * slot_elems * sizeof(uint32_t);
}

extern "C" int iron_tp_allreduce_bf16(const void* part, const void* residual, void* y, int n, int slot_elems,
                                      const void* const* h_peer_buffers, int rank, int world,
                                      unsigned int* d_seq, int* d_status, iron_stream_t stream) {
  if (world <= 0 || world > kTpMaxWorld || rank < 0 || rank >= world) return IRON_ERR_SHAPE;
  if (n <= 0 || (n & 7) || slot_elems < n || (slot_elems & 7)) return IRON_ERR_SHAPE;
  if (!part || !y || !h_peer_buffers || !d_seq) return IRON_ERR_SHAPE;
  if (!aligned16(part) || !aligned16(y) || (residual && !aligned16(residual))) return IRON_ERR_ALIGN;
  TpParams p = {};
  p.part = (const __nv_bfloat16*)part; p.residual = (const __nv_bfloat16*)residual; p.y = (__nv_bfloat16*)y;
  p.n = n; p.slot_elems = slot_elems; p.rank = rank; p.world = world;
  for (int r = 0; r < world; ++r) {
    if (!h_peer_buffers[r] || !aligned16(h_peer_buffers[r])) return IRON_ERR_ALIGN;
    p.peer[r] = static_cast<unsigned char*>(const_cast<void*>(h_peer_buffers[r]));
  }
  p.d_seq = d_seq; p.status = d_status;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(1);
  cfg.blockDim = dim3(512);
  cfg.stream = (cudaStream_t)stream;
  cudaLaunchAttribute attr[1];
  fill_pdl_attr(cfg, attr);
  return cudaLaunchKernelEx(&cfg, tp_allreduce_kernel, p) == cudaSuccess ? IRON_OK : IRON_ERR_LAUNCH;
}

extern "C" int iron_tp_allreduce_tagged_bf16(const void* part, const void* residual, void* y, int n, int slot_elems,
                                             const void* const* h_peer_buffers, int rank, int world,
                                             unsigned int* d_state, int* d_status, iron_stream_t stream) {
  if (world <= 0 || world > kTpMaxWorld || rank < 0 || rank >= world) return IRON_ERR_SHAPE;
  if (n <= 0 || (n & 7) || slot_elems < n || (slot_elems & 7)) return IRON_ERR_SHAPE;
  if (!part || !y || !h_peer_buffers || !d_state) return IRON_ERR_SHAPE;
  if (!aligned16(part) || !aligned16(y) || (residual && !aligned16(residual))) return IRON_ERR_ALIGN;
  TpTaggedParams p = {};
  p.part = (const __nv_bfloat16*)part; p.residual = (const __nv_bfloat16*)residual; p.y = (__nv_bfloat16*)y;
  p.n = n; p.slot_elems = slot_elems; p.rank = rank; p.world = world;
  for (int r = 0; r < world; ++r) {
    if (!h_peer_buffers[r] || !aligned16(h_peer_buffers[r])) return IRON_ERR_ALIGN;
    p.peer[r] = static_cast<unsigned char*>(const_cast<void*>(h_peer_buffers[r]));
  }
  p.state = d_state; p.status = d_status;
  const int groups = n / 4;
  int ctas = (groups + 255) / 256;
  if (ctas > 32) ctas = 32;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(ctas);
  cfg.blockDim = dim3(256);
  cfg.stream = (cudaStream_t)stream;
  cudaLaunchAttribute attr[1];
  fill_pdl_attr(cfg, attr);
  return cudaLaunchKernelEx(&cfg, tp_allreduce_tagged_kernel, p) == cudaSuccess ? IRON_OK : IRON_ERR_LAUNCH;
}
