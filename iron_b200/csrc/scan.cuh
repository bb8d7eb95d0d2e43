// What the selective-scan kernels share: the call's parameters and the step's softplus.
#pragma once
#include "common.cuh"

namespace iron {

struct ScanParams {
  const __nv_bfloat16* xbc;   // (B, rows, width): x (H*P) | B (G*N) | C (G*N)
  const __nv_bfloat16* dt;    // (B, rows, H)
  const float* head;          // (H, 3): dt_bias, A, D
  const float* state;         // (B, H, P, N) or null: zeros
  __nv_bfloat16* y;           // (B, rows, H*P)
  float* final_state;         // (B, H, P, N) or null
  int rows, H, P, G, width;
  int valid;
  const int* d_valid;
  long long xbc_batch, dt_batch, y_batch, state_batch;  // element strides
};

__device__ __forceinline__ float softplus_f32(float v) {
  // logaddexp(0, v) = max(v, 0) + log1p(exp(-|v|))
  return fmaxf(v, 0.f) + log1pf(expf(-fabsf(v)));
}

// The chunked scan on tcgen05 / tensor memory (scan_tc.cu): 128-row chunks, 64-wide heads, 128
// states.  IRON_ERR_UNSUPPORTED when a tensor map cannot describe the call's layout.
int launch_ssd_tc(const ScanParams& p, int batch, cudaStream_t stream, int* d_status);

}  // namespace iron
