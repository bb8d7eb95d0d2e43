"""Launch wrappers: torch CUDA tensors in, one C-ABI call on the current stream, tensors out.

torch is plumbing here (device memory and streams); every arithmetic result comes from
``libiron_b200.so``.  There is no CPU path: a tensor that is not on a CUDA device raises.
"""

from __future__ import annotations

import math

import torch

from . import _lib
from ._lib import call

EW = dict(silu=0, add=1, mul=2, axpy=3, silu_mul=4, row_add=5, row_mul=6, sigmoid=7, gelu_sig=8)


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
         _ptr(v_cache), H, G, D, _stream())
    return q_out


def rms_norm(x, weight=None, out=None, *, eps=1e-5, valid=None, d_valid=None):
    _bf16(x, weight)
    cols = x.shape[-1]
    rows = x.numel() // cols
    if out is None:
        out = torch.empty_like(x)
    call("iron_rmsnorm_bf16", _ptr(x), _ptr(weight), _ptr(out), rows, cols, float(eps),
         rows if valid is None else valid, _ptr(d_valid), _stream())
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
    """Greedy draw: first index of the maximum, written to ``token_out[*d_out_index]``."""
    _bf16(logits)
    call("iron_argmax_bf16", _ptr(logits), logits.numel(), _ptr(token_out), _ptr(d_out_index),
         _ptr(carry_token), _ptr(carry_position), _ptr(workspace), _stream())
    return token_out


def mha_decode_plan(batch, H, G, D, kv_len_hint, device, nsplit=None):
    """Pick a split count and allocate (zeroed) the workspace it needs."""
    lib = _lib.load()
    if nsplit is None:
        nsplit = lib.iron_mha_decode_splits(batch, G, kv_len_hint)
    nbytes = lib.iron_mha_decode_workspace_bytes(batch, H, G, D, nsplit)
    return nsplit, torch.zeros(nbytes, dtype=torch.uint8, device=device)


def mha_decode(Q, K, V, out=None, *, kv_valid=None, d_kv_valid=None, per_batch=False,
               kv_valid_add=0, window=None, scale=None, nsplit=1, workspace=None,
               kv_interleaved=True):
    """One query per (batch, head) over the first ``kv_valid`` keys.

    ``Q`` (B, H, D) or (H, D).  ``K``/``V``: (B?, S, G, D) when ``kv_interleaved`` else
    (B?, G, S, D).
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
    scale = 1.0 / math.sqrt(D) if scale is None else float(scale)
    call("iron_mha_decode_bf16", _ptr(Q), _ptr(K), _ptr(V), _ptr(out), B, H, G, D, S,
         batch_stride, seq_stride, head_stride, S if kv_valid is None else int(kv_valid),
         _ptr(d_kv_valid), 1 if per_batch else 0, int(kv_valid_add),
         -1 if window is None else int(window), scale, int(nsplit), _ptr(workspace),
         0 if workspace is None else workspace.numel(), _stream())
    return out
