/*
 * iron_b200 -- C ABI of the B200 (sm_100a) operator library.
 *
 * The reference (amd/IRON) has no C FFI: its device boundary is the Python operator
 * class (`Operator.__call__` / `Operator.step`, iron/common/declare/operator.py:126-136,
 * :619-637) whose `build()`/`sequence()` halves lower to AIE designs.  On B200 those
 * halves become kernel-launch wrappers that call the entry points declared here, one
 * per kernel family.  Each comment names the reference operator the entry replaces.
 *
 * Conventions
 *   - every pointer is a CUDA device pointer unless its name starts with `h_`;
 *   - bf16 tensors are dense, row-major, 16-byte aligned at their base;
 *   - `stream` is a `cudaStream_t` passed as `void*` (NULL = the legacy default stream);
 *   - the library allocates nothing: outputs, workspaces and the arena are the caller's;
 *   - every launch is stream-ordered and may be captured in a CUDA graph;
 *   - a `const int* d_*` argument, when non-NULL, overrides the immediate of the same
 *     name with a value read on the device at run time, so a captured graph can be
 *     replayed with new per-call values (the reference's per-call `Value`s,
 *     iron/common/declare/value.py:25-114);
 *   - return value: IRON_OK or a negative IRON_ERR_* code; nothing throws or aborts.
 */
#ifndef IRON_B200_H
#define IRON_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void* iron_stream_t;

enum {
  IRON_OK = 0,
  IRON_ERR_SHAPE = -1,       /* a size the kernel family refuses */
  IRON_ERR_ALIGN = -2,       /* a pointer or row pitch that is not 16-byte aligned */
  IRON_ERR_LAUNCH = -3,      /* the CUDA runtime reported a launch error */
  IRON_ERR_UNSUPPORTED = -4, /* a mode this build does not implement */
  IRON_ERR_WORKSPACE = -5,   /* the workspace given is too small */
  IRON_ERR_TIMEOUT = -6      /* a bounded device-side wait gave up (see status word) */
};

/* Library version and the architecture it was compiled for ("sm_100a"). */
int iron_version(void);
const char* iron_arch(void);

/* Every kernel is launched with the programmatic-stream-serialization attribute, so a
 * kernel's weight prefetch may overlap the tail of the kernel before it (each kernel
 * still waits for its predecessor's results before reading them).  iron_set_pdl(0)
 * turns the attribute off process-wide, e.g. to bisect a scheduling problem. */
void iron_set_pdl(int enabled);

/* A hint for the next GEMV-family or decode-attention launch made by this host thread
 * (iron_gemv_bf16, iron_gemv_swiglu_bf16, iron_decode_qkv_rope_bf16, iron_mha_decode_bf16):
 * `bytes` of device memory at `ptr` (16-byte aligned) that kernels launched *after* it will
 * stream, typically the next projection's weights.  The launch spreads L2 prefetches of that
 * region over its CTAs and does not wait for them, so HBM keeps working while a
 * latency-bound kernel runs.  The hint is consumed by that one launch; it never changes a
 * result.  The reference has no counterpart (its weights stream through shim DMA). */
int iron_prefetch_hint(const void* ptr, long long bytes);

/* ------------------------------------------------------------------------------------
 * GEMV -- replaces iron/operators/gemv.py:79 (`GEMV`, reference :408-417).
 *   y[b, m] = bf16( sum_k A[b / repeat, m, k] * xn[b, k] ),  f32 accumulation.
 * A is (num_matrices, M, K) with num_matrices = batches / repeat, x is (batches, K),
 * y is (batches, M).  Rows >= valid_rows are not written.
 * Fused prologue (norm_mode): 0 none; 1 xn = RMSNorm(x) unweighted; 2 xn = RMSNorm(x)
 * times norm_weight (K,) -- with the two bf16 roundings of
 * iron/common/elementwise.py:676-682.
 * Fused epilogue: residual (batches, M) non-NULL adds it after y's own rounding,
 * y = bf16(bf16(acc) + residual), as `ElementwiseAdd` after `GEMV` would.
 * K must be a multiple of 8 and at most 49152.
 */
int iron_gemv_bf16(const void* A, const void* x, void* y, int M, int K, int batches,
                   int repeat, int valid_rows, int norm_mode, const void* norm_weight,
                   float eps, const void* residual, iron_stream_t stream);

/* Gate/up projection with SwiGLU -- the chain GEMV, GEMV, SiLU, ElementwiseMul of
 * iron/lm/blocks.py:697-699 in one pass over both weight matrices:
 *   y[m] = bf16( bf16(silu(bf16(Wg[m,:] . xn))) * bf16(Wu[m,:] . xn) ).
 * Same prologue options as iron_gemv_bf16.  Wg, Wu are (M, K); x (K,); y (M,).
 */
int iron_gemv_swiglu_bf16(const void* Wg, const void* Wu, const void* x, void* y, int M,
                          int K, int norm_mode, const void* norm_weight, float eps,
                          iron_stream_t stream);

/* Decode-step fused QKV projection -- RMSNorm, the three GEMVs, RoPE on q and k and
 * the two KV-cache writes of iron/lm/blocks.py:627-648 and :486 in one kernel.
 * Wqkv is ((H + 2G) * D, K): q rows, then k rows, then v rows.  angles is the packed
 * RoPE table (positions, D) with cos at even and sin at odd columns
 * (iron/operators/rope.py:58); the row used is `position`.  q_out is (H, D);
 * k_cache and v_cache are (cache_rows, G, D) and row `position` of each is written;
 * `angles` has at least cache_rows rows.  A position given on the device (d_position) is
 * held inside 0 .. cache_rows - 1, so a replay past the end of the caches cannot write
 * outside them; an immediate position outside that range is refused (IRON_ERR_SHAPE) --
 * the reference refuses an out-of-range per-call index before any dispatch
 * (iron/common/graph/compiled.py:972-1001).
 */
int iron_decode_qkv_rope_bf16(const void* Wqkv, const void* x, int K, int norm_mode,
                              const void* norm_weight, float eps, const void* angles,
                              int position, const int* d_position, void* q_out,
                              void* k_cache, void* v_cache, int H, int G, int D,
                              int cache_rows, iron_stream_t stream);

/* ------------------------------------------------------------------------------------
 * Row-wise and element-wise kernels.
 */

/* RMSNorm -- iron/operators/rms_norm.py:10 on WeightedRowwise
 * (iron/common/elementwise.py:619-794): per row n = bf16(x * 1/sqrt(mean(x^2)+eps)),
 * then y = bf16(n * weight) when weight is non-NULL.  x, y (rows, cols); cols % 8 == 0. */
int iron_rmsnorm_bf16(const void* x, const void* weight, void* y, int rows, int cols,
                      float eps, int valid_rows, const int* d_valid_rows,
                      iron_stream_t stream);

/* RMSNorm of x * silu(gate) in one launch -- the SiLU, ElementwiseMul and RMSNorm steps that end
 * a Mamba2 mixer (iron/applications/granite_hybrid/model.py:131-135): g = bf16(x * bf16(silu(gate)))
 * element by element, then RMSNorm of g exactly as iron_rmsnorm_bf16.  x, gate, y (rows, cols);
 * cols % 8 == 0 and cols <= 8192. */
int iron_rmsnorm_gated_bf16(const void* x, const void* gate, const void* weight, void* y,
                            int rows, int cols, float eps, int valid_rows,
                            const int* d_valid_rows, iron_stream_t stream);

/* RoPE -- iron/operators/rope.py:58 (reference :167-184).  x, y (rows, cols); angles
 * (angle_rows, cols) packed cos/sin; row r uses angle row
 * angle_offset + r / (rows / angle_rows).  two_halves != 0 pairs column i with
 * i + cols/2 (the Hugging Face layout), else columns 2i and 2i+1. */
int iron_rope_bf16(const void* x, const void* angles, void* y, int rows, int cols,
                   int angle_rows, int two_halves, int angle_offset,
                   const int* d_angle_offset, int valid_rows, const int* d_valid_rows,
                   iron_stream_t stream);

/* Prompt-chunk RoPE and KV-cache write -- the two RoPE steps and the two bounded cache
 * writes `cache[start : start + C][:rows] = x` of iron/lm/blocks.py:642-644 and :483-484
 * in one pass over a fused projection's output.  qkv is (rows, (H + 2G) * D) with row
 * pitch `pitch` (q heads, k heads, v heads); q is rotated in place, k is rotated into
 * k_cache[start + r] and v copied into v_cache[start + r] (caches (max_seq, G, D)).
 * Row r uses angle row angle_start + r.  d_rows / d_start / d_angle_start override on
 * the device. */
int iron_rope_kv_write_bf16(void* qkv, long long pitch, const void* angles, void* k_cache,
                            void* v_cache, int rows, const int* d_rows, int H, int G, int D,
                            int start, const int* d_start, int angle_start,
                            const int* d_angle_start, iron_stream_t stream);

/* Unary / binary element-wise ops over n bf16 elements (n % 8 == 0 not required).
 * op: see IRON_EW_*.  For the ROW variants b is a row of `cols` elements broadcast
 * over n / cols rows.  Replaces iron/operators/{silu,elementwise_add,elementwise_mul,
 * axpy}.py.  Every result is computed in f32 and rounded once. */
enum {
  IRON_EW_SILU = 0,     /* y = silu(a) */
  IRON_EW_ADD = 1,      /* y = a + b */
  IRON_EW_MUL = 2,      /* y = a * b */
  IRON_EW_AXPY = 3,     /* y = scalar * a + b */
  IRON_EW_SILU_MUL = 4, /* y = bf16(silu(a)) * b  (SiLU then ElementwiseMul) */
  IRON_EW_ROW_ADD = 5,  /* y = a + b[col] */
  IRON_EW_ROW_MUL = 6,  /* y = a * b[col] */
  IRON_EW_SIGMOID = 7,  /* y = 1 / (1 + exp(-a)) */
  IRON_EW_GELU_SIG = 8, /* y = a * sigmoid(1.702 a) */
  IRON_EW_RELU = 9,     /* y = max(a, 0) */
  IRON_EW_TANH = 10,    /* y = tanh(a) */
  IRON_EW_GELU_TANH = 11, /* y = 0.5 a (1 + tanh(sqrt(2/pi) (a + 0.044715 a^3))) */
  IRON_EW_GELU_ERF = 12 /* y = 0.5 a (1 + erf(a / sqrt 2)) */
};
int iron_elementwise_bf16(int op, const void* a, const void* b, void* y, long long n,
                          int cols, float scalar, iron_stream_t stream);

/* Clamp -- iron/operators/clamp.py: y = min(max(x, low), high) with the bounds rounded to
 * bf16 first (exact). */
int iron_clamp_bf16(const void* x, void* y, long long n, float low, float high, iron_stream_t stream);

/* LayerNorm -- iron/operators/layer_norm.py:10 on WeightedRowwise (beta 0): per row
 * n = bf16((x - mean) / sqrt(var + eps)) with the biased variance, then y = bf16(n * weight)
 * when weight is non-NULL.  x, y (rows, cols); cols % 8 == 0. */
int iron_layernorm_bf16(const void* x, const void* weight, void* y, int rows, int cols, float eps,
                        int valid_rows, const int* d_valid_rows, iron_stream_t stream);

/* Softmax -- iron/operators/softmax.py:77 (reference :523-545): per row, over the first
 * `length` columns, y = softmax(v) with v = x (+ addend, f32), then soft_cap * tanh(v / soft_cap)
 * when soft_cap > 0; f32 throughout, y (bf16) rounded once; columns >= length are zeros.
 * x is bf16, or f32 when x_is_f32 != 0 (the operator's input_dtype).  d_length overrides
 * length when non-NULL.  cols % 8 == 0.  The banded form (window, period) is not provided. */
int iron_softmax_bf16(const void* x, int x_is_f32, const float* addend, void* y, int rows, int cols,
                      int length, const int* d_length, float soft_cap, iron_stream_t stream);

/* Copy / Gather -- iron/operators/copy.py:546 (`Copy`, reference :839-902) and :72
 * (`Gather`), exact.  Gathers `nrows` rows of `row_bytes` bytes (multiple of 16):
 *   dst[(dst_row0 + i) * dst_pitch ...] = src[row(i) * src_pitch ...]
 * where row(i) = ids ? clamp(ids[i], 0, src_rows - 1) : src_row0 + i.  d_src_row0 /
 * d_dst_row0 / d_nrows override the immediates when non-NULL; nrows is then the
 * upper bound the grid is sized for. */
int iron_copy_rows(const void* src, void* dst, const int* ids, int nrows,
                   const int* d_nrows, long long row_bytes, long long src_pitch,
                   long long dst_pitch, int src_rows, int src_row0, const int* d_src_row0,
                   int dst_row0, const int* d_dst_row0, iron_stream_t stream);

/* Greedy draw -- the all-zero draw row of iron/operators/sample.py:106, i.e.
 * iron/lm/generation.py:97-99: the first index of the largest logit, exact.
 * logits (n,) bf16.  workspace: iron_argmax_workspace_bytes() bytes, zeroed once by the
 * caller before first use (the kernel leaves it zeroed).  token_out[*d_out_index]
 * (index 0 when d_out_index is NULL) receives the id -- `drawn[position]` of
 * iron/lm/causal.py:340-347; when carry_token / carry_position are non-NULL the id is
 * also stored there and *carry_position is incremented afterwards, which is how a
 * captured decode loop carries (token, position + 1) to its next replay
 * (iron/lm/causal.py:348).  out_rows > 0 is the length of token_out: an index outside
 * 0 .. out_rows - 1 writes nothing, and when d_out_index and carry_position are the same
 * word (the row written is the carried position, a decoder's loop) the position stops
 * growing at out_rows, so a loop replayed past the end of its caches stays inside its
 * buffers; out_rows <= 0 means no bound. */
size_t iron_argmax_workspace_bytes(int n);
int iron_argmax_bf16(const void* logits, int n, int* token_out, const int* d_out_index,
                     int out_rows, int* carry_token, int* carry_position, void* workspace,
                     iron_stream_t stream);

/* The greedy draw when the output head is split by vocabulary rows across ranks (the
 * reference keeps the head whole on one device; a later row of its plan shards it): each
 * rank reduces its rows' logits to one 64-bit key -- the value made monotone in the high
 * word, the complement of the GLOBAL row index (index_offset + local index) in the low word
 * -- with iron_argmax_key_bf16; the keys of all ranks are gathered (any all-gather) and
 * iron_argmax_pick takes their maximum, which is the first index of the largest logit over
 * the whole vocabulary (iron/lm/generation.py:97-99), and stores and carries it exactly as
 * iron_argmax_bf16 does.  key_out and keys are 8-byte aligned. */
int iron_argmax_key_bf16(const void* logits, int n, int index_offset, void* key_out, void* workspace,
                         iron_stream_t stream);
int iron_argmax_pick(const void* keys, int count, int* token_out, const int* d_out_index, int out_rows,
                     int* carry_token, int* carry_position, iron_stream_t stream);

/* The same greedy draw for callers that cannot give the library a workspace.  It has no
 * counterpart in the reference.  A caller may be unable to allocate device memory at all: a
 * thread that must never enter the CUDA allocator (which can lock or synchronise), a plugin
 * inside a runtime that owns every byte of device memory and offers no hook to ask for more,
 * or code running where allocation is not permitted.  Here the cross-block scratch is a
 * fixed array inside the library (a few kilobytes per GPU, held until the process exits), so
 * the call takes inputs and outputs only and performs no allocation of any kind.
 *   - n may be at most iron_argmax_noalloc_max_n() (4 194 304); larger n returns
 *     IRON_ERR_WORKSPACE.
 *   - The first call on each device looks up the array's device address; make that first
 *     call outside any stream capture.
 *   - All calls on a device share the one array: two calls whose kernels could overlap on
 *     the GPU (different streams, no ordering between them) race.  Calls on one stream,
 *     or otherwise ordered, are safe; each call resets the part that must start at zero. */
int iron_argmax_noalloc_max_n(void);
int iron_argmax_bf16_noalloc(const void* logits, int n, int* token_out, const int* d_out_index,
                             int* carry_token, int* carry_position, iron_stream_t stream);

/* ------------------------------------------------------------------------------------
 * GEMM -- replaces iron/operators/gemm.py:143 (`GEMM`, reference :696-702) and
 * iron/operators/flm/gemm/op.py:128 (`ProjectionGEMM`, reference :1335-1346, output
 * stage iron/operators/flm/gemm/design.py:92-112), which `F.linear` records for a
 * prompt chunk (iron/functional.py:50-60).
 *   C = epilogue( bf16( A[:valid_rows, :valid_k] @ B[:valid_k] ) ) (+ residual)
 * A is (M, K) row-major with row pitch lda.  B is (N, K) when b_col_maj (a checkpoint's
 * (out, in) weight) else (K, N), row pitch ldb.  C is (M, N), or (N, M) when c_col_maj,
 * pitch ldc; bf16, or f32 when out_f32 (no epilogue then).  Accumulation is f32 in
 * tensor memory (tcgen05.mma), rounded once.  epilogue: 0 none, 1 x*sigmoid(1.702x),
 * 2 silu, 3 sigmoid, applied to the rounded product as the reference does.  residual
 * (same layout as C, bf16) is added after the rounding, as ElementwiseAdd would.
 * Rows >= valid_rows (d_valid_rows overrides on the device) are neither computed nor
 * written.  lda, ldb multiples of 8; bases 16-byte aligned.  d_status (optional device
 * int) receives IRON_ERR_TIMEOUT if a bounded pipeline wait gave up.
 */
int iron_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, int lda,
                   int ldb, int ldc, int b_col_maj, int c_col_maj, int valid_rows,
                   const int* d_valid_rows, int valid_k, int epilogue, const void* residual,
                   int out_f32, int* d_status, iron_stream_t stream);

/* The fused q/k/v projection of a prompt chunk with RoPE and the cache write in its output
 * stage -- iron/lm/blocks.py:472-499 records a ProjectionGEMM, RoPE steps on q and k and the
 * bounded cache copies; here rows [0, valid_rows) of A (M, K) times Wqkv ((H + 2G) D, K)^T,
 * each output rounded to bf16, then per head: q rotated into qkv (rows ldc apart), k rotated
 * into k_cache[start + row], v copied into v_cache[start + row] (caches (S, G, D)), with the
 * angle row angle_start + row and the roundings of iron_rope_kv_write_bf16, bit for bit.
 * Returns IRON_ERR_UNSUPPORTED for shapes the CTA-pair GEMM does not take (one row tile):
 * the caller then runs iron_gemm_bf16 and iron_rope_kv_write_bf16.  D is 64 or 128. */
int iron_gemm_qkv_rope_bf16(const void* A, const void* Wqkv, void* qkv, int M, int K, int lda, int ldb,
                            int ldc, int valid_rows, const void* angles, void* k_cache, void* v_cache,
                            int H, int G, int D, int start, int angle_start, int* d_status,
                            iron_stream_t stream);

/* Gate/up projection with SwiGLU for a block of rows -- the chain ProjectionGEMM,
 * ProjectionGEMM, SiLU, ElementwiseMul that `GatedMLP.body` records for a prompt chunk
 * (iron/lm/blocks.py:697-699) in one pass over both weight matrices:
 *   C[m, n] = bf16( bf16(silu(bf16(A[m,:] . Wg[n,:]))) * bf16(A[m,:] . Wu[n,:]) ).
 * A is (M, K) with pitch lda, Wg and Wu are (N, K) with pitch ldb (checkpoint layout), C is
 * (M, N) with pitch ldc.  One tensor-memory accumulator holds 128 columns of both products,
 * so gate and up never travel through HBM.  valid_rows / d_valid_rows as in iron_gemm_bf16. */
int iron_gemm_swiglu_bf16(const void* A, const void* Wg, const void* Wu, void* C, int M, int N,
                          int K, int lda, int ldb, int ldc, int valid_rows,
                          const int* d_valid_rows, int* d_status, iron_stream_t stream);

/* ------------------------------------------------------------------------------------
 * The projections of a BATCHED decode step (1 to 64 sequences, one row each), with the layer's
 * RMSNorm, RoPE and cache write folded into them -- iron/lm/blocks.py's `Attention.body` and
 * `GatedMLP.body` chains RMSNorm, ProjectionGEMM, RoPE, cache write ... ProjectionGEMM + residual,
 * RMSNorm, ProjectionGEMM x 2, SiLU, ElementwiseMul, ProjectionGEMM + residual as five launches
 * a layer instead of eight.
 *
 * iron_gemm_rows_bf16: C (rows, N; pitch ldc) = X (rows <= 64, K; pitch ldx) . W^T, W (N, K; pitch
 * ldw) as a checkpoint stores it; the weights cross HBM once.
 *   W2 != NULL        the gated pair: C = bf16(silu(bf16(X . W^T))) * bf16(X . W2^T), no residual.
 *   residual          (rows, N; pitch ldc) added after the product's rounding.
 *   d_rowsq_out       with a residual: this call also leaves, per row, the sum of squares of the
 *                     bf16 values it wrote, as iron_gemm_rows_parts(rows, N, K, 0) partial sums in
 *                     fixed slots of a float[64][320] buffer (row-major; no atomics).
 *   norm_weight, d_rowsq_in, rowsq_parts, eps
 *                     RMSNorm of X before the product (iron/operators/rms_norm.py): the sums the
 *                     call that PRODUCED X left; X is normalised on its way into shared memory with
 *                     the norm's own two roundings, bf16(bf16(x / rms) * weight).  K % 64 == 0.
 * IRON_ERR_UNSUPPORTED for a product this kernel does not take (more than 296 tiles of 128 rows).
 *
 * iron_gemm_rows_qkv_rope_bf16: the q/k/v projection of such a step (Wqkv ((H + 2G) D, K), rows
 * q | k | v), the optional folded RMSNorm as above, then per row RoPE of q and k with the angle
 * row (interleaved cos, sin; two-halves pairing) of d_positions[row], q to q_out (rows, H, D),
 * k and v to row d_positions[row] of that sequence's caches ((rows, S, G, D), sequences
 * kv_batch_stride elements apart).  D 64 or 128, H D and G D multiples of 128. */
int iron_gemm_rows_parts(int rows, int N, int K, int gated);
int iron_gemm_rows_bf16(const void* X, const void* W, const void* W2, void* C, const void* residual,
                        int rows, int N, int K, int ldx, int ldw, int ldc, const void* norm_weight,
                        const float* d_rowsq_in, int rowsq_parts, float eps, float* d_rowsq_out,
                        int* d_status, iron_stream_t stream);
int iron_gemm_rows_qkv_rope_bf16(const void* X, const void* Wqkv, int rows, int K, int ldx, int ldw,
                                 const void* norm_weight, const float* d_rowsq_in, int rowsq_parts,
                                 float eps, const void* angles, const int* d_positions, void* q_out,
                                 void* k_cache, void* v_cache, long long kv_batch_stride, int H, int G,
                                 int D, int S, int* d_status, iron_stream_t stream);

/* ------------------------------------------------------------------------------------
 * One decode step's attention, o_proj and residual add of a layer in one launch -- the
 * reference's steps MHA (iron/operators/mha.py:191 as iron/lm/blocks.py:487-502 calls it: one
 * query row per head over the cache rows 0 .. position, grouped heads, an optional window),
 * the o_proj GEMV (iron/operators/gemv.py:79, iron/lm/blocks.py:646-648) and the residual add
 * (iron/lm/blocks.py:723-728):
 *   y = bf16( x + bf16( Wo . att ) ),   att = bf16( softmax(scale * q K^T) V ) per head.
 * One thread-block cluster of eight CTAs per KV group: before the previous kernel's results
 * are needed its CTAs stage their rows of the group's column block of Wo and their slice of
 * the cached keys and values in shared memory; they exchange the attention partials over
 * distributed shared memory and leave a float32 partial of y per group in `scratch`; for
 * each eighth of the rows the last CTA to arrive adds the partials in group order.
 * q (H, D) as iron_decode_qkv_rope_bf16 leaves it, Wo (E, H * D), x and y (E), the caches
 * (cache_rows, G, D) with row `position` already written (immediate, or *d_position held
 * inside the caches); keys 0 .. position attend (the last `window + 1` when window >= 0).
 * scratch: iron_decode_attn_oproj_scratch_bytes(E, G) bytes, zeroed once by the caller (the
 * kernel leaves its counters zero); launches ordered on one stream may share it.
 * iron_decode_attn_oproj_supported() is the number of cache rows of a group one CTA holds at
 * a time (longer contexts run in several passes), 0 when a CTA's rows of Wo do not fit one
 * SM's shared memory or there are more groups than clusters the GPU holds at once (the entry
 * point then returns IRON_ERR_UNSUPPORTED and the two separate kernels serve).  A copy that
 * does not land within 2 s sets *d_status to IRON_ERR_TIMEOUT; nothing hangs.
 * iron_decode_attn_oproj_trace is a diagnostic: a device buffer of 16 x (8 G) 64-bit words
 * that later launches on the current device fill with each CTA's phase timestamps in
 * nanoseconds (NULL turns it off again). */
size_t iron_decode_attn_oproj_scratch_bytes(int E, int G);
int iron_decode_attn_oproj_supported(int E, int H, int G, int D);
void iron_decode_attn_oproj_trace(void* d_trace);
int iron_decode_attn_oproj_bf16(const void* q, const void* Wo, const void* x, int position,
                                const int* d_position, const void* k_cache, const void* v_cache,
                                void* y, int E, int H, int G, int D, int cache_rows, int window,
                                float scale, void* scratch, int* d_status, iron_stream_t stream);

/* ------------------------------------------------------------------------------------
 * Mamba2.
 */

/* Selective scan -- iron/operators/selective_scan.py:46 (reference :367-383).  Per batch
 * entry and row t < valid_rows: x = xbc[t, :H*P] as (H, P); B, C = the two halves of
 * xbc[t, H*P:], each (G, N), head h reading group h / (H/G);
 *   step = softplus(dt[t, h] + dt_bias[h]);  state = exp(step * A[h]) * state + step * x (x) B;
 *   y[t] = state . C + D[h] * x,
 * float32 throughout, y rounded once to bf16.  head is (H, 3) f32 = (dt_bias, A, D);
 * state / final_state are (batch, H, P, N) f32 (state NULL = zeros, final_state NULL =
 * not wanted).  xbc (batch, rows, H*P + 2*G*N), dt (batch, rows, H), y (batch, rows, H*P),
 * all dense.  Rows >= valid_rows of y are zeros.  N is 16, 32, 64 or 128; P % 8 == 0.
 * The reference operator has no batch axis: batch > 1 is the independent-sequence axis.
 * Calls of 32 rows or more with P = 64 and N of 64 or 128 run in the chunked form on the
 * tensor cores (64-row chunks: scores C B^T, decay-masked scores times x, C times the
 * carried state, the state update, as bf16 products with float32 accumulation and a float32
 * state): the same function within the operator's tolerance (iron/operators/
 * selective_scan.py:353-356), not bit for bit the step-by-step kernel.  With 128 states and at
 * least 128 rows the chunks are 128 rows and the four products run as tcgen05.mma with
 * tensor-memory accumulators (TMA-fed operands; the float32 operands enter as a bf16 head and
 * remainder).  iron_set_scan_chunked(mode), or IRON_SCAN_CHUNKED in the environment: 2 (default)
 * tcgen05 where the shape fits, 1 warp MMAs only, 0 every call step by step.
 * iron_selective_scan_status_word names the device word that receives IRON_ERR_TIMEOUT when a
 * bounded pipeline wait of the tcgen05 kernel gives up (NULL: none; per device). */
void iron_set_scan_chunked(int mode);
void iron_selective_scan_status_word(int* d_status);
int iron_selective_scan_bf16(const void* xbc, const void* dt, const void* head,
                             const void* state, void* y, void* final_state, int batch,
                             int rows, int heads, int head_dim, int state_size, int groups,
                             int valid_rows, const int* d_valid_rows, iron_stream_t stream);

/* Short causal depth-wise convolution -- iron/functional.py:147-180 (`F.causal_conv1d`) with
 * the bias of iron/lm/causal.py:163 and the SiLU of
 * iron/applications/granite_hybrid/model.py:128 optionally fused:
 *   y[t, c] = sum_k taps[k, c] * xx[t + k, c],  xx = history (K-1 rows) ++ x,
 * each product and each partial sum rounded to bf16 as the recorded RowwiseMul /
 * ElementwiseAdd steps do; decode_order != 0 sums the newest tap first (the one-row form).
 * new_history receives the K-1 rows ending the valid run (may alias history).  x, y
 * (batch, rows, channels); taps (K, channels); K is 2, 3 or 4; channels % 8 == 0. */
int iron_causal_conv1d_bf16(const void* x, const void* taps, const void* bias,
                            const void* history, void* new_history, void* y, int batch,
                            int rows, int channels, int kernel, int valid_rows,
                            const int* d_valid_rows, int decode_order, int silu,
                            iron_stream_t stream);

/* ------------------------------------------------------------------------------------
 * Attention.
 */

/* One-query ("packed") attention over a KV cache -- iron/operators/mha.py:191 with
 * seq_len == 1 (reference :1073-1116), as iron/lm/blocks.py:491-499 calls it for a
 * decode step: O[b,h,:] = softmax(scale * Q[b,h,:] . K[b, :n, h / (H/G), :]) . V.
 * Q, O are (batch, H, D).  K and V share the element strides given: the cache layout
 * (max_seq, G, D) of iron/lm/blocks.py:460 is seq_stride = G*D, head_stride = D.
 * n = kv_valid, or d_kv_valid[b * d_kv_valid_stride] + kv_valid_add when d_kv_valid is
 * non-NULL; clamped to kv_max.  window < 0 attends all n keys, else the query's own
 * and the `window` before it.  D is 64, 128 or 256.  The keys are split over a
 * thread-block cluster of nsplit CTAs (1, 2, 4 or 8; iron_mha_decode_splits suggests
 * one); partial results meet in distributed shared memory, so no workspace is needed.
 * stable_prefix != 0 promises that the kernel launched just before this one on the
 * stream wrote at most row n-1 of K and V (true of a decode step), which lets the key
 * loads start before that kernel has finished.
 * Grouped heads (H > G, D 64 or 128) take tensor-core forms that choose their own split: from
 * 16 (sequence, KV head) pairs on, one CTA a pair with the keys split over a cluster while the
 * pairs do not fill the machine; below that, every CTA holds its share of a cache of up to
 * about 100 K key rows x pairs in shared memory and the last CTA of a pair folds the partials
 * through a scratch the library owns (1.2 MB per GPU, held until exit): calls of that form that
 * OVERLAP on one GPU (two streams) would race; calls of one stream do not.
 * IRON_MHA_DECODE_RESIDENT=0 / IRON_MHA_DECODE_TC=0 keep the cluster kernel described first. */
int iron_mha_decode_splits(int batch, int G, int kv_len_hint);
int iron_mha_decode_bf16(const void* Q, const void* K, const void* V, void* O, int batch,
                         int H, int G, int D, int kv_max, long long kv_batch_stride,
                         long long kv_seq_stride, long long kv_head_stride, int kv_valid,
                         const int* d_kv_valid, int d_kv_valid_stride, int kv_valid_add,
                         int window, float scale, int nsplit, int stable_prefix,
                         iron_stream_t stream);

/* Multi-query attention -- iron/operators/mha.py:191 with seq_len > 1 (reference
 * :1073-1116), as iron/lm/blocks.py:491-499 calls it for a prompt chunk.  The q_tokens
 * queries are the last rows of the kv_tokens keys (position of query i is
 * kv_tokens - q_tokens + i); causal keeps keys <= position, window >= 0 keeps keys
 * within `window` positions (both sides when not causal).  Output rows in
 * [q_tokens, q_rows) are written as zeros and keys >= kv_tokens are masked
 * (iron/operators/mha.py:1076-1096).  Q, O and K/V (K and V share theirs) each have
 * element strides (batch, row, head): a (rows, heads, D) layout has row stride heads*D
 * and head stride D; Q may be a view into a wider fused projection (larger row stride).
 * d_q_tokens / d_kv_tokens (+ kv_tokens_add) override the bounds on the device.
 * D is 64 or 128. */
int iron_mha_prefill_bf16(const void* Q, const void* K, const void* V, void* O, int batch,
                          int H, int G, int D, int q_rows, int kv_rows,
                          long long q_batch_stride, long long q_row_stride,
                          long long q_head_stride, long long o_batch_stride,
                          long long o_row_stride, long long o_head_stride,
                          long long kv_batch_stride,
                          long long kv_row_stride, long long kv_head_stride, int q_tokens,
                          const int* d_q_tokens, int kv_tokens, const int* d_kv_tokens,
                          int kv_tokens_add, int causal, int window, float scale,
                          iron_stream_t stream);

/* The device word that receives IRON_ERR_TIMEOUT when a bounded pipeline wait of the
 * tensor-memory prompt attention gives up (NULL: none).  Applies to the launches that follow;
 * set it once per process to a word the caller reads after synchronising.  No counterpart
 * in the reference. */
void iron_mha_prefill_status_word(int* d_status);

/* ------------------------------------------------------------------------------------
 * Tensor-parallel all-reduce of a small bf16 vector through peer memory, fused with the
 * residual add that follows it -- the exchange step after the row-parallel o_proj and
 * down_proj when a decoder is sharded over GPUs (the reference is single-device; its
 * residual add is iron/lm/blocks.py:386-391):
 *   y = bf16( bf16( sum over ranks of part_r ) + residual ),  partials added in rank order.
 * Every rank owns one buffer of iron_tp_buffer_bytes(world, slot_elems) bytes that all
 * ranks can address (peer-mapped, zeroed once); h_peer_buffers is a HOST array with the
 * `world` device addresses of those buffers as THIS rank sees them, own buffer included.
 * d_seq is a device counter private to the rank, zeroed once; every call advances it, and
 * all ranks must make the same sequence of calls.  One launch per rank: it stores its
 * partial into every rank's buffer, raises a flag there, waits (at most 2 s) for every
 * rank's flag in its own buffer and reduces.  A wait that gives up writes IRON_ERR_TIMEOUT
 * to *d_status and the kernel finishes with the data it has.  n % 8 == 0, n <= slot_elems,
 * world <= 8. */
size_t iron_tp_buffer_bytes(int world, int slot_elems);
int iron_tp_allreduce_bf16(const void* part, const void* residual, void* y, int n, int slot_elems,
                           const void* const* h_peer_buffers, int rank, int world,
                           unsigned int* d_seq, int* d_status, iron_stream_t stream);

/* The same exchange folded into the GEMVs on either side of it, so that it costs no launch of
 * its own.  Each call below attaches the exchange to the NEXT GEMV-family launch this host thread
 * makes (iron_gemv_bf16, iron_gemv_swiglu_bf16, iron_decode_qkv_rope_bf16) and is consumed by it,
 * whatever that launch returns.
 *   iron_tp_push_next: the next iron_gemv_bf16 (no residual, one batch) stores every rounded row
 *     into slot [parity][rank] of EVERY rank's buffer instead of y (y must still be a valid
 *     pointer), as one 32-bit word: the bf16 value and a 16-bit tag of the exchange's number.  A
 *     word arrives whole, so the tag says its value is there: no fence, no flag, no count.
 *   iron_tp_pull_next: the next launch takes its activation vector not from x but from the
 *     exchange: every CTA reads all ranks' rows, re-reading words whose tag is not yet this
 *     exchange's (at most 2 s, then IRON_ERR_TIMEOUT in *d_status and zero for what is missing),
 *     and builds x = bf16(bf16(sum over ranks, in rank order) + residual); one CTA also stores it
 *     to x_out (the next residual).  Any fused RMSNorm then applies to that x.  The last CTA to
 *     finish advances d_state to the next exchange.
 * Buffers, h_peer_buffers, rank, world and slot_elems are as for iron_tp_allreduce_bf16 (the
 * tagged words use the buffers' whole length, that kernel's bf16 slots the first half); d_state is
 * eight device words private to the rank, zeroed once (the exchange's sequence number, a CTA
 * count).  A push and the pull that consumes it form one exchange; all ranks make the same
 * sequence of exchanges, and an engine uses either these or iron_tp_allreduce_bf16 on one set
 * of buffers, not both.  The tensors named here must outlive the launch that consumes the call.
 * No counterpart in the reference (it is single-device). */
/* The all-reduce as one launch of many CTAs without a fence or a flag: the values travel as the
 * tagged 32-bit words described above (the same slots and d_state as iron_tp_push_next /
 * iron_tp_pull_next), every CTA stores its run of the elements to every rank and re-reads the own
 * buffer until every rank's words of that run carry this exchange's tag (at most 2 s, then
 * IRON_ERR_TIMEOUT in *d_status and zero for what is missing).  For the few rows of a decode
 * batch (n = rows x hidden <= slot_elems); arguments as iron_tp_allreduce_bf16 with d_state in
 * place of d_seq. */
int iron_tp_allreduce_tagged_bf16(const void* part, const void* residual, void* y, int n, int slot_elems,
                                  const void* const* h_peer_buffers, int rank, int world,
                                  unsigned int* d_state, int* d_status, iron_stream_t stream);
int iron_tp_push_next(const void* const* h_peer_buffers, int rank, int world, int slot_elems,
                      unsigned int* d_state, int* d_status);
int iron_tp_pull_next(const void* const* h_peer_buffers, int rank, int world, int slot_elems,
                      unsigned int* d_state, int* d_status, const void* residual, void* x_out);

/* ------------------------------------------------------------------------------------
 * Batched decode: every row of the batch is another sequence at its own position with its
 * own KV cache -- the reference runs such sequences one Session at a time
 * (iron/lm/session.py:138-144); the per-row arithmetic is that of iron/lm/blocks.py:642-644
 * (RoPE), :483-486 (cache write) and iron/operators/sample.py:148 (greedy draw).
 *
 * iron_rope_kv_scatter_bf16: qkv is (rows, (H + 2G) * D) with row pitch `pitch` (elements).
 * Row r is rotated with angle row d_positions[r]; q goes to q_out (rows, H, D) dense, k and v
 * into row d_positions[r] of the caches of sequence r, which start kv_batch_stride elements
 * apart (each (S, G, D)).  Positions are clamped to [0, S - 1].
 *
 * iron_argmax_rows_bf16: logits is (rows, n) with row pitch `pitch`; for every row the first
 * index of the maximum goes to drawn[r * S + positions[r]] and tokens[r], and positions[r]
 * advances by one. */
int iron_rope_kv_scatter_bf16(const void* qkv, long long pitch, const void* angles, void* q_out,
                              void* k_cache, void* v_cache, long long kv_batch_stride, int rows,
                              const int* d_positions, int H, int G, int D, int S,
                              iron_stream_t stream);
int iron_argmax_rows_bf16(const void* logits, long long pitch, int rows, int n, int* tokens,
                          int* positions, int* drawn, int S, iron_stream_t stream);

/* Temperature / top-k draw -- iron/operators/sample.py:106 with a non-zero draw row, the
 * device side of iron/lm/generation.py:24-94 (`Sampler`).  The reference's arithmetic
 * (`sample_ref`) lives in mlir-aie, outside its tree: the rule here is this library's own,
 * stated in iron_b200/lm/generation.py, whose host Sampler it matches token for token.
 * Per row r at position p = positions[r]: the draw row draws[(r * S + p) * 4 ..] holds the
 * temperature's f32 bits, top_k (clamped to iron_sample_k_max()), and the low 32 / high 21
 * bits of a 53-bit uniform; an all-zero row, temperature 0 or top_k 1 is the greedy draw.
 * The token goes to drawn[r * S + p] and tokens[r]; positions[r] becomes p + 1 (the carry of
 * iron_argmax_rows_bf16).  logits (rows, pitch >= n) bf16. */
int iron_sample_k_max(void);
int iron_sample_rows_bf16(const void* logits, long long pitch, int rows, int n, const int* draws,
                          int* tokens, int* positions, int* drawn, int S, iron_stream_t stream);

/* ------------------------------------------------------------------------------------
 * One whole greedy decode step as one persistent kernel -- replaces the decode version the
 * reference records per call, iron/lm/causal.py:248-287 (embedding gather, per layer
 * iron/lm/blocks.py:438-470: RMSNorm, q/k/v GEMV, RoPE, cache write, packed attention,
 * o_proj + residual, RMSNorm, gate/up GEMV, SiLU, product, down_proj + residual; final
 * RMSNorm, head, argmax iron/operators/sample.py:148).  The same arithmetic and roundings
 * as the separate entry points above (dot products in another summation order), in one
 * cooperative launch, one CTA per SM, whose phases are separated by a bounded grid barrier.
 * Every warp streams its share of the weights of ALL phases through a private
 * shared-memory ring filled by tiled TMA copies, so the weight stream does not stop
 * between projections.  Batch 1, one GPU.
 *   layer_ptrs : DEVICE array of L x 9 pointers per layer, in this order (16-byte aligned):
 *                ln1 (E), wqkv ((H+2G)*D x E), wo (E x H*D), ln2 (E), wg (F x E),
 *                wu (F x E), wd (E x F), k cache (S x G x D), v cache (S x G x D)
 *   maps       : DEVICE copy (64-byte aligned) of the tensor maps
 *                iron_decode_step_encode_maps wrote for the same pointers
 *   values     : device int32[2] = (token, position); left as (drawn token, position + 1)
 *   drawn      : device int32[S]; drawn[position] receives the token
 *   xa, xb (E), act (F), logits (V): bf16 transients, 16-byte aligned; on return xa holds
 *                the residual stream after the last layer and logits the step's logits
 *   workspace  : iron_decode_step_workspace_bytes(E, H, G, D) bytes, 16-byte aligned, zeroed
 *                once by the caller.  Byte 128 holds an int status word: 0, or
 *                IRON_ERR_TIMEOUT after a wait gave up (2 s); it is sticky until the caller
 *                zeroes it, and a step launched while it is set returns early.
 * D is 64 or 128; E, F and H*D are multiples of 32 and at most 8192; V is a multiple of 8;
 * L is at most 64.  The launch is cooperative (every CTA resident); it may be captured in
 * a CUDA graph.
 *
 * iron_decode_step_encode_maps runs on the host and launches nothing: it describes every
 * weight matrix to the TMA engine.  h_layer_ptrs is a HOST array with the same L x 9 device
 * pointers as layer_ptrs; h_maps_out is a HOST buffer of iron_decode_step_maps_bytes(L)
 * bytes that the caller then copies to device memory. */
size_t iron_decode_step_workspace_bytes(int E, int H, int G, int D);
size_t iron_decode_step_maps_bytes(int L);
int iron_decode_step_encode_maps(const void* const* h_layer_ptrs, int L, int E, int F, int H, int G,
                                 int D, int V, const void* head, void* h_maps_out);
int iron_decode_step_bf16(const void* const* layer_ptrs, const void* maps, int L, int E, int F,
                          int H, int G, int D, int V, int S, const void* embed, const void* head,
                          const void* final_norm, const void* angles, float eps, float scale,
                          int window, int* values, int* drawn, void* xa, void* xb, void* act,
                          void* logits, void* workspace, iron_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* IRON_B200_H */
