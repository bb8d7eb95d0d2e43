"""Launch wrappers: torch CUDA tensors in, one C-ABI call on the current stream, tensors out.

torch is plumbing here (device memory and streams); every arithmetic result comes from
``libiron_b200.so``.  There is no CPU path: a tensor that is not on a CUDA device raises.
"""

from __future__ import annotations

import math

import torch

from . import _lib
from ._lib import call

EW = dict(silu=0, add=1, mul=2, axpy=3, silu_mul=4, row_add=5, row_mul=6, sigmoid=7, gelu_sig=8,
          relu=9, tanh=10, gelu_tanh=11, gelu_erf=12)


def _ptr(t: torch.Tensor | None) -> int | None:
    if t is None:
        return None
    if not t.is_cuda:
        raise RuntimeError("iron_b200 kernels take CUDA tensors only (no CPU fallback)")
    if not t.is_contiguous():
        raise ValueError("iron_b200 kernels take contiguous tensors")
    return t.data_ptr()


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _bf16(*ts):
    for t in ts:
        if t is not None and t.dtype != torch.bfloat16:
            raise TypeError(f"expected bfloat16, got {t.dtype}")


def gemv(A, x, out=None, *, repeat=1, valid=None, norm_weight=None, norm=False, eps=1e-5,
         residual=None):
    """``out[b] = A[b // repeat] @ x[b]``; optional fused RMSNorm of ``x`` and residual add."""
    _bf16(A, x, norm_weight, residual)
    M, K = A.shape[-2], A.shape[-1]
    batches = 1 if x.dim() == 1 else x.shape[0]
    if out is None:
        out = torch.empty((M,) if x.dim() == 1 else (batches, M), dtype=torch.bfloat16, device=A.device)
    mode = 2 if norm_weight is not None else (1 if norm else 0)
    call("iron_gemv_bf16", _ptr(A), _ptr(x), _ptr(out), M, K, batches, repeat,
         M if valid is None else valid, mode, _ptr(norm_weight), float(eps), _ptr(residual), _stream())
    return out


def gemv_swiglu(Wg, Wu, x, out=None, *, norm_weight=None, norm=False, eps=1e-5):
    """``silu(Wg @ x) * (Wu @ x)`` with the chain's bf16 roundings, one pass."""
    _bf16(Wg, Wu, x, norm_weight)
    M, K = Wg.shape
    if out is None:
        out = torch.empty((M,), dtype=torch.bfloat16, device=x.device)
    mode = 2 if norm_weight is not None else (1 if norm else 0)
    call("iron_gemv_swiglu_bf16", _ptr(Wg), _ptr(Wu), _ptr(x), _ptr(out), M, K, mode,
         _ptr(norm_weight), float(eps), _stream())
    return out


def decode_qkv_rope(Wqkv, x, angles, k_cache, v_cache, q_out, *, H, G, D, position=0,
                    d_position=None, norm_weight=None, norm=False, eps=1e-5):
    """RMSNorm + fused QKV GEMV + RoPE + KV-cache write at ``position`` (decode step)."""
    _bf16(Wqkv, x, angles, k_cache, v_cache, q_out, norm_weight)
    mode = 2 if norm_weight is not None else (1 if norm else 0)
    call("iron_decode_qkv_rope_bf16", _ptr(Wqkv), _ptr(x), Wqkv.shape[1], mode, _ptr(norm_weight),
         float(eps), _ptr(angles), int(position), _ptr(d_position), _ptr(q_out), _ptr(k_cache),
         _ptr(v_cache), H, G, D, min(k_cache.shape[0], angles.shape[0]), _stream())
    return q_out


def attn_oproj_supported(E: int, H: int, G: int, D: int) -> int:
    """Cache rows of a KV group one CTA of the one-launch attention + o_proj holds at a time;
    0: the shape does not run on it."""
    return _lib.load().iron_decode_attn_oproj_supported(E, H, G, D)


def attn_oproj_scratch(E: int, G: int, device) -> torch.Tensor:
    return torch.zeros(_lib.load().iron_decode_attn_oproj_scratch_bytes(E, G), dtype=torch.uint8, device=device)


def decode_attn_oproj(q, Wo, x, k_cache, v_cache, y, *, G, scratch, position=0, d_position=None, window=None,
                      scale=None, status=None):
    """One decode step's attention over the cache rows 0 .. position, o_proj and the residual
    add in one launch: ``y = x + Wo @ attention(q, K, V)``.  ``q`` (H, D); caches (S, G, D)."""
    _bf16(q, Wo, x, k_cache, v_cache, y)
    H, D = q.shape[-2], q.shape[-1]
    call("iron_decode_attn_oproj_bf16", _ptr(q), _ptr(Wo), _ptr(x), int(position), _ptr(d_position),
         _ptr(k_cache), _ptr(v_cache), _ptr(y), x.numel(), H, G, D, k_cache.shape[0],
         -1 if window is None else int(window), 1.0 / math.sqrt(D) if scale is None else float(scale),
         _ptr(scratch), _ptr(status), _stream())
    return y


def rms_norm(x, weight=None, out=None, *, eps=1e-5, valid=None, d_valid=None):
    _bf16(x, weight)
    cols = x.shape[-1]
    rows = x.numel() // cols
    if out is None:
        out = torch.empty_like(x)
    call("iron_rmsnorm_bf16", _ptr(x), _ptr(weight), _ptr(out), rows, cols, float(eps),
         rows if valid is None else valid, _ptr(d_valid), _stream())
    return out


def rms_norm_gated(x, gate, weight=None, out=None, *, eps=1e-5, valid=None, d_valid=None):
    """RMSNorm of ``x * silu(gate)`` (each step rounded as the separate operators round) in one launch."""
    _bf16(x, gate, weight)
    if x.shape != gate.shape:
        raise ValueError(f"x {tuple(x.shape)} and gate {tuple(gate.shape)} differ in shape")
    cols = x.shape[-1]
    rows = x.numel() // cols
    if out is None:
        out = torch.empty_like(x)
    call("iron_rmsnorm_gated_bf16", _ptr(x), _ptr(gate), _ptr(weight), _ptr(out), rows, cols, float(eps),
         rows if valid is None else valid, _ptr(d_valid), _stream())
    return out


def layer_norm(x, weight=None, out=None, *, eps=1e-5, valid=None, d_valid=None):
    """Each row minus its mean over its standard deviation (biased), rounded, times ``weight``."""
    _bf16(x, weight)
    cols = x.shape[-1]
    rows = x.numel() // cols
    if out is None:
        out = torch.empty_like(x)
    call("iron_layernorm_bf16", _ptr(x), _ptr(weight), _ptr(out), rows, cols, float(eps),
         rows if valid is None else valid, _ptr(d_valid), _stream())
    return out


def softmax(x, out=None, *, addend=None, soft_cap=None, length=None, d_length=None):
    """Softmax over the first ``length`` columns of each row of ``x`` (bf16 or float32), zeros past them."""
    if x.dtype not in (torch.bfloat16, torch.float32):
        raise TypeError(f"softmax input is bf16 or float32, not {x.dtype}")
    if addend is not None and addend.dtype != torch.float32:
        raise TypeError("the addend is float32")
    cols = x.shape[-1]
    rows = x.numel() // cols
    if out is None:
        out = torch.empty(x.shape, dtype=torch.bfloat16, device=x.device)
    call("iron_softmax_bf16", _ptr(x), int(x.dtype == torch.float32), _ptr(addend), _ptr(out), rows, cols,
         cols if length is None else int(length), _ptr(d_length), float(soft_cap or 0.0), _stream())
    return out


def clamp(x, low, high, out=None):
    """``x`` clamped to ``[low, high]``, the bounds rounded to bf16 (exact)."""
    _bf16(x)
    if out is None:
        out = torch.empty_like(x)
    call("iron_clamp_bf16", _ptr(x), _ptr(out), x.numel(), float(low), float(high), _stream())
    return out


def rope(x, angles, out=None, *, angle_rows=None, two_halves=True, angle_offset=0,
         d_angle_offset=None, valid=None, d_valid=None):
    """Rotate ``x`` (rows, cols) by ``angles``; row r uses angle row offset + r // (rows/angle_rows)."""
    _bf16(x, angles)
    rows, cols = x.shape
    if angle_rows is None:
        angle_rows = angles.shape[0]
    if out is None:
        out = torch.empty_like(x)
    call("iron_rope_bf16", _ptr(x), _ptr(angles), _ptr(out), rows, cols, angle_rows,
         int(bool(two_halves)), int(angle_offset), _ptr(d_angle_offset),
         rows if valid is None else valid, _ptr(d_valid), _stream())
    return out


def elementwise(op: str, a, b=None, out=None, *, scalar=0.0):
    _bf16(a, b)
    if out is None:
        out = torch.empty_like(a)
    cols = b.numel() if (b is not None and op.startswith("row_")) else 0
    call("iron_elementwise_bf16", EW[op], _ptr(a), _ptr(b), _ptr(out), a.numel(), cols,
         float(scalar), _stream())
    return out


def copy_rows(src, dst, *, ids=None, nrows, row_bytes, src_pitch=None, dst_pitch=None,
              src_rows=0, src_row0=0, dst_row0=0, d_nrows=None, d_src_row0=None, d_dst_row0=None):
    """Move ``nrows`` rows of ``row_bytes`` bytes; rows picked by ``ids`` (clipped) when given."""
    src_pitch = row_bytes if src_pitch is None else src_pitch
    dst_pitch = row_bytes if dst_pitch is None else dst_pitch
    if ids is not None and ids.dtype != torch.int32:
        raise TypeError("ids must be int32")
    call("iron_copy_rows", _ptr(src), _ptr(dst), _ptr(ids), nrows, _ptr(d_nrows), row_bytes,
         src_pitch, dst_pitch, src_rows, src_row0, _ptr(d_src_row0), dst_row0, _ptr(d_dst_row0),
         _stream())
    return dst


def argmax_workspace(device) -> torch.Tensor:
    n = _lib.load().iron_argmax_workspace_bytes(0)
    return torch.zeros(n, dtype=torch.uint8, device=device)


def argmax(logits, token_out, workspace, *, d_out_index=None, carry_token=None,
           carry_position=None):
    """Greedy draw: first index of the maximum, written to ``token_out[*d_out_index]`` (an
    index past ``token_out``'s end writes nothing and the carried position stops there)."""
    _bf16(logits)
    call("iron_argmax_bf16", _ptr(logits), logits.numel(), _ptr(token_out), _ptr(d_out_index),
         token_out.numel(), _ptr(carry_token), _ptr(carry_position), _ptr(workspace), _stream())
    return token_out


def argmax_key(logits, key_out, workspace, *, index_offset=0):
    """One shard's candidate for the greedy draw: ``key_out`` (one int64) receives the 64-bit
    key of the largest of ``logits``, whose rows start at global row ``index_offset``."""
    _bf16(logits)
    call("iron_argmax_key_bf16", _ptr(logits), logits.numel(), int(index_offset), _ptr(key_out), _ptr(workspace),
         _stream())
    return key_out


def argmax_pick(keys, token_out, *, d_out_index=None, carry_token=None, carry_position=None):
    """The draw from every shard's key: the largest names the token (first index of the maximum)."""
    call("iron_argmax_pick", _ptr(keys), keys.numel(), _ptr(token_out), _ptr(d_out_index), token_out.numel(),
         _ptr(carry_token), _ptr(carry_position), _stream())
    return token_out


def mha_decode_splits(batch, G, kv_len_hint) -> int:
    """The cluster size (key splits) suggested for a context of ``kv_len_hint`` keys."""
    return _lib.load().iron_mha_decode_splits(batch, G, kv_len_hint)


def mha_decode(Q, K, V, out=None, *, kv_valid=None, d_kv_valid=None, per_batch=False,
               kv_valid_add=0, window=None, scale=None, nsplit=None, kv_interleaved=True,
               stable_prefix=False):
    """One query per (batch, head) over the first ``kv_valid`` keys.

    ``Q`` (B, H, D) or (H, D).  ``K``/``V``: (B?, S, G, D) when ``kv_interleaved`` else
    (B?, G, S, D).  ``stable_prefix``: only the newest cache row was written by the
    kernel launched just before (a decode step).
    """
    _bf16(Q, K, V)
    q3 = Q if Q.dim() == 3 else Q.unsqueeze(0)
    B, H, D = q3.shape
    k4 = K if K.dim() == 4 else K.unsqueeze(0)
    if kv_interleaved:
        S, G = k4.shape[1], k4.shape[2]
        seq_stride, head_stride = G * D, D
    else:
        G, S = k4.shape[1], k4.shape[2]
        seq_stride, head_stride = D, S * D
    batch_stride = S * G * D if k4.shape[0] > 1 or B == 1 else 0
    if out is None:
        out = torch.empty_like(Q)
    if nsplit is None:
        nsplit = mha_decode_splits(B, G, S if kv_valid is None else int(kv_valid))
    scale = 1.0 / math.sqrt(D) if scale is None else float(scale)
    call("iron_mha_decode_bf16", _ptr(Q), _ptr(K), _ptr(V), _ptr(out), B, H, G, D, S,
         batch_stride, seq_stride, head_stride, S if kv_valid is None else int(kv_valid),
         _ptr(d_kv_valid), 1 if per_batch else 0, int(kv_valid_add),
         -1 if window is None else int(window), scale, int(nsplit), int(bool(stable_prefix)),
         _stream())
    return out


EPILOGUES = dict(none=0, gelu=1, silu=2, sigmoid=3)


def gemm(A, B, out=None, *, b_col_maj=False, c_col_maj=False, valid=None, d_valid=None,
         valid_k=None, epilogue="none", residual=None, out_f32=False, status=None):
    """``epilogue(bf16(A @ B))`` on the tensor cores (tcgen05, f32 accumulation in TMEM).

    ``A`` (M, K); ``B`` (N, K) when ``b_col_maj`` (a checkpoint's (out, in) weight) else
    (K, N); the result is (M, N), or (N, M) when ``c_col_maj``.
    """
    _bf16(A, B, residual)
    M, Kd = A.shape
    N = B.shape[0] if b_col_maj else B.shape[1]
    if (B.shape[1] if b_col_maj else B.shape[0]) != Kd:
        raise ValueError(f"gemm: A {tuple(A.shape)} and B {tuple(B.shape)} do not chain")
    if out is None:
        out = torch.empty((N, M) if c_col_maj else (M, N),
                          dtype=torch.float32 if out_f32 else torch.bfloat16, device=A.device)
    if residual is not None and (tuple(residual.shape) != tuple(out.shape) or residual.stride() != out.stride()):
        # the kernel walks the residual with the output's pitch
        raise ValueError(f"gemm: residual {tuple(residual.shape)} (strides {residual.stride()}) is not laid out "
                         f"as the output {tuple(out.shape)} (strides {out.stride()})")
    call("iron_gemm_bf16", _ptr(A), _ptr(B), _ptr(out), M, N, Kd, A.stride(0), B.stride(0),
         out.stride(0), int(b_col_maj), int(c_col_maj), M if valid is None else int(valid),
         _ptr(d_valid), Kd if valid_k is None else int(valid_k), EPILOGUES[epilogue],
         _ptr(residual), int(out_f32), _ptr(status), _stream())
    return out


def gemm_swiglu(A, Wg, Wu, out=None, *, valid=None, d_valid=None, status=None):
    """``bf16(silu(bf16(A @ Wg.T))) * bf16(A @ Wu.T)`` in one tensor-core pass.

    ``A`` (M, K); ``Wg`` and ``Wu`` (N, K) as a checkpoint stores them; the result is (M, N)."""
    _bf16(A, Wg, Wu)
    M, Kd = A.shape
    N = Wg.shape[0]
    if Wg.shape != Wu.shape or Wg.shape[1] != Kd:
        raise ValueError(f"gemm_swiglu: A {tuple(A.shape)}, Wg {tuple(Wg.shape)}, Wu {tuple(Wu.shape)} do not chain")
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=A.device)
    call("iron_gemm_swiglu_bf16", _ptr(A), _ptr(Wg), _ptr(Wu), _ptr(out), M, N, Kd, A.stride(0), Wg.stride(0),
         out.stride(0), M if valid is None else int(valid), _ptr(d_valid), _ptr(status), _stream())
    return out


_PREFILL_STATUS: dict = {}


def prefill_status(device=None):
    """The device word the tensor-memory prompt attention reports a given-up wait in
    (``IRON_ERR_TIMEOUT``); allocated once per device and handed to the library."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    if dev not in _PREFILL_STATUS:
        _PREFILL_STATUS[dev] = torch.zeros(1, dtype=torch.int32, device=dev)
    _lib.load().iron_mha_prefill_status_word(_PREFILL_STATUS[dev].data_ptr())
    return _PREFILL_STATUS[dev]


def mha_prefill(Q, K, V, out=None, *, q_tokens=None, d_q_tokens=None, kv_tokens=None,
                d_kv_tokens=None, kv_tokens_add=0, causal=True, window=None, scale=None,
                heads_interleaved=True, kv_interleaved=True, q_row_stride=None):
    """Attention of ``Q``'s rows over ``K``/``V``, the queries the keys' last rows.

    ``Q`` (rows, H, D) when ``heads_interleaved`` else (H, rows, D); ``K``/``V`` (rows, G, D)
    when ``kv_interleaved`` else (G, rows, D); an optional leading batch axis on all.
    """
    _bf16(Q, K, V)
    if Q.device not in _PREFILL_STATUS:
        prefill_status(Q.device)
    if q_row_stride is not None:
        # Q is a strided view (rows, H, D) into a wider fused projection: rows are
        # `q_row_stride` elements apart and O is dense (rows, H, D).
        rows, H, D = Q.shape
        kv_rows, G = K.shape[0], K.shape[1]
        if out is None:
            out = torch.empty((rows, H, D), dtype=torch.bfloat16, device=Q.device)
        scale = 1.0 / math.sqrt(D) if scale is None else float(scale)
        if not (K.is_contiguous() and V.is_contiguous() and out.is_contiguous()):
            raise ValueError("K, V and the output must be contiguous")
        call("iron_mha_prefill_bf16", Q.data_ptr(), _ptr(K), _ptr(V), _ptr(out), 1, H, G, D, rows,
             kv_rows, 0, int(q_row_stride), D, 0, H * D, D, 0, G * D, D,
             rows if q_tokens is None else int(q_tokens), _ptr(d_q_tokens),
             kv_rows if kv_tokens is None else int(kv_tokens), _ptr(d_kv_tokens), int(kv_tokens_add),
             int(bool(causal)), -1 if window is None else int(window), scale, _stream())
        return out
    q4 = Q if Q.dim() == 4 else Q.unsqueeze(0)
    k4 = K if K.dim() == 4 else K.unsqueeze(0)
    B = q4.shape[0]
    if heads_interleaved:
        rows, H, D = q4.shape[1:]
        q_row, q_head = H * D, D
    else:
        H, rows, D = q4.shape[1:]
        q_row, q_head = D, rows * D
    if kv_interleaved:
        kv_rows, G = k4.shape[1], k4.shape[2]
        kv_row, kv_head = G * D, D
    else:
        G, kv_rows = k4.shape[1], k4.shape[2]
        kv_row, kv_head = D, kv_rows * D
    if out is None:
        out = torch.empty_like(Q)
    scale = 1.0 / math.sqrt(D) if scale is None else float(scale)
    call("iron_mha_prefill_bf16", _ptr(Q), _ptr(K), _ptr(V), _ptr(out), B, H, G, D, rows, kv_rows,
         rows * H * D, q_row, q_head, rows * H * D, q_row, q_head, kv_rows * G * D, kv_row, kv_head,
         rows if q_tokens is None else int(q_tokens), _ptr(d_q_tokens),
         kv_rows if kv_tokens is None else int(kv_tokens), _ptr(d_kv_tokens), int(kv_tokens_add),
         int(bool(causal)), -1 if window is None else int(window), scale, _stream())
    return out


def rope_kv_write(qkv, angles, k_cache, v_cache, *, rows, H, G, D, start=0, angle_start=None,
                  d_rows=None, d_start=None, d_angle_start=None):
    """Rotate q in place and write rotated k and v rows into the caches at ``start``."""
    _bf16(qkv, angles, k_cache, v_cache)
    call("iron_rope_kv_write_bf16", _ptr(qkv), qkv.stride(0), _ptr(angles), _ptr(k_cache),
         _ptr(v_cache), int(rows), _ptr(d_rows), H, G, D, int(start), _ptr(d_start),
         int(start if angle_start is None else angle_start), _ptr(d_angle_start), _stream())
    return qkv


def gemm_qkv_rope(x, wqkv, qkv, angles, k_cache, v_cache, *, H, G, D, start=0, angle_start=None, status=None) -> bool:
    """The fused q/k/v projection of a prompt chunk: ``x @ wqkv.T`` with RoPE and the cache
    write in the GEMM's output stage (q into ``qkv``, k and v into the caches at ``start``).
    Returns False, having launched nothing, for shapes only the two separate kernels take."""
    _bf16(x, wqkv, qkv, angles, k_cache, v_cache)
    rc = _lib.load().iron_gemm_qkv_rope_bf16(
        _ptr(x), _ptr(wqkv), _ptr(qkv), x.shape[0], x.shape[1], x.stride(0), wqkv.stride(0), qkv.stride(0),
        x.shape[0], _ptr(angles), _ptr(k_cache), _ptr(v_cache), H, G, D, int(start),
        int(start if angle_start is None else angle_start), _ptr(status), _stream())
    if rc == -4:
        return False
    if rc != 0:
        raise _lib.IronError("iron_gemm_qkv_rope_bf16", rc)
    return True


def selective_scan(xbc, dt, head, state=None, *, heads, head_dim, state_size, groups=1, valid=None,
                   d_valid=None, want_final=True, y=None, final=None):
    """Mamba2's recurrence; returns ``(y bf16, final f32)``.  A leading batch axis is optional.
    ``final`` may be ``state`` itself: a state is read whole before any of it is written."""
    _bf16(xbc, dt, y)
    batched = xbc.dim() == 3
    B = xbc.shape[0] if batched else 1
    rows = xbc.shape[-2]
    inner = heads * head_dim
    if y is None:
        y = torch.empty((*xbc.shape[:-1], inner), dtype=torch.bfloat16, device=xbc.device)
    shape = (B, heads, head_dim, state_size) if batched else (heads, head_dim, state_size)
    if final is None and want_final:
        final = torch.empty(shape, dtype=torch.float32, device=xbc.device)
    if head.dtype != torch.float32 or (state is not None and state.dtype != torch.float32) or (
            final is not None and final.dtype != torch.float32):
        raise TypeError("head and state are float32")
    call("iron_selective_scan_bf16", _ptr(xbc), _ptr(dt), _ptr(head), _ptr(state), _ptr(y), _ptr(final),
         B, rows, heads, head_dim, state_size, groups, rows if valid is None else int(valid),
         _ptr(d_valid), _stream())
    return y, final


def causal_conv1d(x, taps, *, bias=None, history=None, new_history=None, out=None, valid=None,
                  d_valid=None, decode_order=False, silu=False):
    """Depth-wise causal conv over ``x`` (rows, C) or (B, rows, C) with ``taps`` (K, C)."""
    _bf16(x, taps, bias, history, new_history)
    B = x.shape[0] if x.dim() == 3 else 1
    rows, C = x.shape[-2], x.shape[-1]
    if out is None:
        out = torch.empty_like(x)
    call("iron_causal_conv1d_bf16", _ptr(x), _ptr(taps), _ptr(bias), _ptr(history), _ptr(new_history),
         _ptr(out), B, rows, C, taps.shape[0], rows if valid is None else int(valid), _ptr(d_valid),
         int(bool(decode_order)), int(bool(silu)), _stream())
    return out


def prefetch_hint(*tensors) -> None:
    """Tell the next GEMV-family / decode-attention launch which weights come after it.

    ``tensors`` must be adjacent in memory (one arena run); the launch prefetches the whole
    run into L2.
    """
    ts = [t for t in tensors if t is not None]
    if not ts:
        return
    lo = min(t.data_ptr() for t in ts)
    hi = max(t.data_ptr() + t.numel() * t.element_size() for t in ts)
    call("iron_prefetch_hint", lo, hi - lo)


def decode_step_workspace(E: int, H: int, G: int, D: int, device) -> torch.Tensor:
    """Zeroed workspace of the one-kernel decode step (barrier, status word, partials)."""
    n = _lib.load().iron_decode_step_workspace_bytes(E, H, G, D)
    return torch.zeros(n, dtype=torch.uint8, device=device)


def decode_step_table(layers, device) -> torch.Tensor:
    """The device table of per-layer pointers ``decode_step`` reads: for every layer
    ln1, wqkv, wo, ln2, wg, wu, wd, k cache, v cache (cache tensors of one sequence)."""
    rows = []
    for l in layers:
        rows.append([l[n].data_ptr() for n in ("ln1", "wqkv", "wo", "ln2", "wg", "wu", "wd", "k", "v")])
    return torch.tensor(rows, dtype=torch.int64).to(device)


def decode_step_maps(table: torch.Tensor, *, E, F, H, G, D, V, head) -> torch.Tensor:
    """The device copy of the TMA tensor maps of every weight matrix ``table`` points to."""
    import numpy as np

    host = np.ascontiguousarray(table.cpu().numpy())
    L = host.shape[0]
    n = _lib.load().iron_decode_step_maps_bytes(L)
    out = np.zeros(n, dtype=np.uint8)
    call("iron_decode_step_encode_maps", host.ctypes.data, L, E, F, H, G, D, V, _ptr(head), out.ctypes.data)
    # cudaMalloc'ed storage is 256-byte aligned: the maps need 64
    return torch.from_numpy(out).to(table.device)


def decode_step(table, maps, *, L, E, F, H, G, D, V, S, embed, head, final_norm, angles, eps, scale,
                window, values, drawn, xa, xb, act, logits, workspace):
    """One greedy decode step in one cooperative launch (token and position in ``values``)."""
    _bf16(embed, head, final_norm, angles, xa, xb, act, logits)
    call("iron_decode_step_bf16", _ptr(table), _ptr(maps), L, E, F, H, G, D, V, S, _ptr(embed), _ptr(head),
         _ptr(final_norm), _ptr(angles), float(eps), float(scale), -1 if window is None else int(window),
         _ptr(values), _ptr(drawn), _ptr(xa), _ptr(xb), _ptr(act), _ptr(logits), _ptr(workspace),
         _stream())


def decode_step_status(workspace: torch.Tensor) -> int:
    """The step kernel's status word (0, or IRON_ERR_TIMEOUT after a barrier wait gave up)."""
    return int(workspace[128:132].view(torch.int32).item())


def rope_kv_scatter(qkv, angles, q_out, k_cache, v_cache, positions, *, H, G, D):
    """Per-sequence RoPE and cache write of a batched decode step.

    ``qkv`` (rows, (H + 2G) * D); ``positions`` int32 (rows,) on the device; ``k_cache`` and
    ``v_cache`` (rows, S, G, D); ``q_out`` (rows, H, D) dense."""
    _bf16(qkv, angles, q_out, k_cache, v_cache)
    rows, S = qkv.shape[0], k_cache.shape[1]
    call("iron_rope_kv_scatter_bf16", _ptr(qkv), qkv.stride(0), _ptr(angles), _ptr(q_out), _ptr(k_cache),
         _ptr(v_cache), k_cache.stride(0), rows, _ptr(positions), H, G, D, S, _stream())


ROWSQ_PITCH = 320   # floats between the rows of a sums-of-squares buffer (iron_gemm_rows_bf16)


def rowsq_buffer(device=None):
    """The (64, 320) float32 buffer a projection leaves its rows' sums of squares in."""
    return torch.zeros((64, ROWSQ_PITCH), dtype=torch.float32, device=device or "cuda")


def gemm_rows_parts(rows: int, N: int, K: int, gated: bool = False) -> int:
    """How many partial sums per row ``gemm_rows(..., rowsq_out=...)`` of this shape leaves
    (0: the weight-streaming kernel does not take the shape)."""
    return int(_lib.load().iron_gemm_rows_parts(rows, N, K, int(gated)))


def _norm_args(norm_weight, rowsq_in, rowsq_parts):
    if (norm_weight is None) != (rowsq_in is None):
        raise ValueError("a folded RMSNorm takes both its weight and the producing call's sums of squares")
    if rowsq_in is not None and (rowsq_in.dtype != torch.float32 or rowsq_in.shape != (64, ROWSQ_PITCH)):
        raise TypeError("rowsq buffers are (64, 320) float32")
    return _ptr(norm_weight), _ptr(rowsq_in), int(rowsq_parts)


def gemm_rows(X, W, out=None, *, W2=None, residual=None, norm_weight=None, rowsq_in=None, rowsq_parts=0,
              eps=1e-5, rowsq_out=None, status=None):
    """``X @ W.T`` for a decode batch (up to 64 rows) against weights as stored, optionally with
    the RMSNorm before it folded in (``norm_weight``, ``rowsq_in``, ``rowsq_parts``: the sums of
    squares the call that produced ``X`` left through its ``rowsq_out``), as the gated pair
    (``W2``), or with a residual."""
    _bf16(X, W)
    rows, Kd = X.shape
    N = W.shape[0]
    if W.shape[1] != Kd or (W2 is not None and W2.shape != W.shape):
        raise ValueError(f"gemm_rows: X {tuple(X.shape)} and W {tuple(W.shape)} do not chain")
    if out is None:
        out = torch.empty((rows, N), dtype=torch.bfloat16, device=X.device)
    if residual is not None and (residual.shape != out.shape or residual.stride(0) != out.stride(0)):
        raise ValueError("the residual has the output's shape and pitch")
    if rowsq_out is not None and (rowsq_out.dtype != torch.float32 or rowsq_out.shape != (64, ROWSQ_PITCH)):
        raise TypeError("rowsq buffers are (64, 320) float32")
    nw, sq, parts = _norm_args(norm_weight, rowsq_in, rowsq_parts)
    call("iron_gemm_rows_bf16", _ptr(X), _ptr(W), _ptr(W2), _ptr(out), _ptr(residual), rows, N, Kd, X.stride(0),
         W.stride(0), out.stride(0), nw, sq, parts, float(eps), _ptr(rowsq_out), _ptr(status), _stream())
    return out


def gemm_rows_qkv_rope(X, Wqkv, angles, q_out, k_cache, v_cache, positions, *, H, G, D, norm_weight=None,
                       rowsq_in=None, rowsq_parts=0, eps=1e-5, status=None):
    """The q/k/v projection of a batched decode step with RoPE and the cache write (and
    optionally the RMSNorm before it) folded in; arguments as ``rope_kv_scatter``."""
    _bf16(X, Wqkv, angles, q_out, k_cache, v_cache)
    rows, Kd = X.shape
    if Wqkv.shape != ((H + 2 * G) * D, Kd):
        raise ValueError(f"gemm_rows_qkv_rope: Wqkv {tuple(Wqkv.shape)} is not ({(H + 2 * G) * D}, {Kd})")
    if positions.dtype != torch.int32:
        raise TypeError("positions are int32")
    nw, sq, parts = _norm_args(norm_weight, rowsq_in, rowsq_parts)
    call("iron_gemm_rows_qkv_rope_bf16", _ptr(X), _ptr(Wqkv), rows, Kd, X.stride(0), Wqkv.stride(0), nw, sq, parts,
         float(eps), _ptr(angles), _ptr(positions), _ptr(q_out), _ptr(k_cache), _ptr(v_cache), k_cache.stride(0),
         H, G, D, k_cache.shape[1], _ptr(status), _stream())


def sample_k_max() -> int:
    """The largest top-k the device draws."""
    return _lib.load().iron_sample_k_max()


def sample_rows(logits, draws, tokens, positions, drawn):
    """Per row: the token its draw row (``draws[row, position]``: temperature bits, top_k, a
    53-bit uniform) picks from ``logits[row]``; ``drawn[row, position]`` and ``tokens[row]``
    receive it and ``positions[row]`` advances.  All-zero draw rows are greedy."""
    _bf16(logits)
    rows, n = (1, logits.shape[0]) if logits.dim() == 1 else logits.shape
    pitch = logits.stride(0) if logits.dim() == 2 else n
    S = drawn.shape[-1]
    for t in (draws, tokens, positions, drawn):
        if t.dtype != torch.int32:
            raise TypeError("draws, tokens, positions and drawn are int32")
    if draws.numel() != rows * S * 4:
        raise ValueError(f"draws holds {draws.numel()} words, not {rows} x {S} x 4")
    call("iron_sample_rows_bf16", _ptr(logits), pitch, rows, n, _ptr(draws), _ptr(tokens), _ptr(positions),
         _ptr(drawn), S, _stream())


def argmax_rows(logits, tokens, positions, drawn):
    """Greedy draw per row; ``drawn`` (rows, S) int32, ``tokens`` and ``positions`` int32 (rows,)."""
    _bf16(logits)
    rows, n = logits.shape
    call("iron_argmax_rows_bf16", _ptr(logits), logits.stride(0), rows, n, _ptr(tokens), _ptr(positions),
         _ptr(drawn), drawn.shape[1], _stream())


def tp_buffer_bytes(world: int, slot_elems: int) -> int:
    return _lib.load().iron_tp_buffer_bytes(world, slot_elems)


def tp_push_next(*, peer_buffers, slot_elems, rank, world, state, status=None) -> None:
    """The next ``gemv`` call stores its rows into every rank's exchange buffer instead of ``y``."""
    call("iron_tp_push_next", peer_buffers, rank, world, slot_elems, _ptr(state), _ptr(status))


def tp_pull_next(*, peer_buffers, slot_elems, rank, world, state, status=None, residual=None, x_out=None) -> None:
    """The next GEMV-family call takes ``x = sum over ranks + residual`` from the exchange (and
    stores it to ``x_out``) instead of reading its ``x`` argument."""
    _bf16(residual, x_out)
    call("iron_tp_pull_next", peer_buffers, rank, world, slot_elems, _ptr(state), _ptr(status),
         _ptr(residual), _ptr(x_out))


def tp_allreduce_tagged(part, y, *, residual=None, peer_buffers, slot_elems, rank, world, state, status=None):
    """``tp_allreduce`` as one launch of many CTAs over tagged 32-bit words (no fence, no flag);
    ``state``: the rank's eight device words of ``tp_push_next`` / ``tp_pull_next``."""
    _bf16(part, y)
    call("iron_tp_allreduce_tagged_bf16", _ptr(part), _ptr(residual), _ptr(y), part.numel(), slot_elems,
         peer_buffers, rank, world, _ptr(state), _ptr(status), _stream())
    return y


def tp_allreduce(part, y, *, residual=None, peer_buffers, slot_elems, rank, world, seq, status=None):
    """Sum ``part`` over the tensor-parallel ranks through peer memory, add ``residual``.

    ``peer_buffers``: a ctypes array of ``world`` device addresses (every rank's exchange
    buffer as this rank maps it); ``seq``: this rank's device sequence counter."""
    _bf16(part, y)
    call("iron_tp_allreduce_bf16", _ptr(part), _ptr(residual), _ptr(y), part.numel(), slot_elems,
         peer_buffers, rank, world, _ptr(seq), _ptr(status), _stream())
    return y
