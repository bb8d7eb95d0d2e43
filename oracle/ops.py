"""CPU oracle: numpy restatements of the reference's per-operator ``reference()`` methods.

TEST INFRASTRUCTURE ONLY.  Nothing under ``iron_b200/`` imports this package; it is the
checker for ``tests/``, ``__graft_entry__.smoke()`` and the ``cpu_baseline`` /
``--impl reference`` legs of ``bench.py``.

The reference (amd/IRON) cannot be imported here: every operator module imports the
un-vendored ``aie`` (mlir-aie ``1.4.6.dev15+ge5a3fa1``, requirements.txt:9) at top level.
Each function below restates the arithmetic of the in-repo ``reference()`` it cites
(path:line within the reference tree); where the arithmetic lives in mlir-aie
(RMSNorm, SiLU, add/mul/axpy contracts, ``rope_ref``) the published formula is restated
and pinned by the reference's own formula tests and model goldens (see
``tests/test_oracle_golden.py``).

Convention everywhere (AGENTS.md:169-171): inputs are bf16, arithmetic is float32, each
operator rounds its output to bf16 once.
"""

from __future__ import annotations

import numpy as np
from ml_dtypes import bfloat16

f32 = np.float32


def _f(x) -> np.ndarray:
    return np.asarray(x).astype(f32)


# ---------------------------------------------------------------------------------------
# GEMV / GEMM


def gemv(A, B, repeat: int = 1):
    """``C = A @ B``, one product per batch -- iron/operators/gemv.py:408-417."""
    A, B = np.asarray(A), np.asarray(B)
    if repeat > 1:
        A = np.repeat(A.reshape(-1, *A.shape[-2:]), repeat, axis=0)
    a, b = _f(A), _f(B)
    if A.ndim == 3:
        b = b.reshape(A.shape[0], A.shape[2], 1)
        return np.matmul(a, b).reshape(A.shape[0], A.shape[1]).astype(A.dtype)
    return (a @ b.reshape(A.shape[-1])).astype(A.dtype)


def gemm(A, B, *, b_col_maj=False, c_col_maj=False, valid_k=None, output_dtype=bfloat16):
    """``A @ B`` over the first ``valid_k`` of K -- iron/operators/gemm.py:696-702."""
    K = np.asarray(A).shape[1]
    valid_k = K if valid_k is None else valid_k
    a = _f(A)[:, :valid_k]
    b = _f(np.asarray(B).T if b_col_maj else B)[:valid_k]
    C = np.matmul(b.T, a.T) if c_col_maj else np.matmul(a, b)
    return C.astype(output_dtype)


def gemm_bound(A, B, *, b_col_maj=False, c_col_maj=False, units=2.0):
    """GEMM's admitted error, ``units * 2^-8 * |A| @ |B|`` -- iron/operators/gemm.py:704-735."""
    a = _f(A)
    b = _f(np.asarray(B).T if b_col_maj else B)
    err = units * (np.abs(a) @ np.abs(b)) * 2.0**-8
    return err.T if c_col_maj else err


def sigmoid_rounded(x):
    """``1/(1+exp(-x))`` in float32, rounded to ``x``'s dtype -- iron/operators/flm/gemm/design.py:109-112."""
    x = np.asarray(x)
    return (1 / (1 + np.exp(-_f(x)))).astype(x.dtype)


def projection_gemm(A, B, *, b_col_maj=True, epilogue="none"):
    """``epilogue(bf16(A @ B))`` -- iron/operators/flm/gemm/op.py:1335-1346, design.py:92-106."""
    A = np.asarray(A)
    b = np.asarray(B).T if b_col_maj else np.asarray(B)
    C = np.matmul(_f(A), _f(b)).astype(A.dtype)
    if epilogue == "gelu":
        C = C * sigmoid_rounded(f32(1.702) * C)
    elif epilogue == "silu":
        C = C * sigmoid_rounded(C)
    elif epilogue == "sigmoid":
        C = sigmoid_rounded(C)
    elif epilogue != "none":
        raise ValueError(epilogue)
    return C


# ---------------------------------------------------------------------------------------
# Row-wise / element-wise


def rms_norm(x, weight=None, eps: float = 1e-5):
    """Row RMS norm, rounded, then times ``weight``, rounded again.

    iron/operators/rms_norm.py:10-20 on WeightedRowwise, iron/common/elementwise.py:676-682
    (the kernel contract is mlir-aie's ``norm.rms_norm_eps``; the formula
    ``x / sqrt(mean(x^2) + eps) * w`` is pinned in-repo by
    iron/tests/lm/test_modules.py:204-206).
    """
    x = np.asarray(x)
    xf = _f(x)
    inv = f32(1.0) / np.sqrt(np.mean(xf * xf, axis=-1, keepdims=True, dtype=f32) + f32(eps))
    normed = (xf * inv).astype(x.dtype)
    if weight is None:
        return normed
    return (_f(normed) * _f(weight)).astype(x.dtype)


def rope(x, angles, two_halves: bool = True):
    """Rotate each row by its packed cos/sin row -- iron/operators/rope.py:167-184.

    ``angles`` holds cos at even and sin at odd columns; row ``r`` of ``x`` uses angle
    row ``r // (rows / angle_rows)``.  The formula is the one written out in
    iron/tests/operators/test_rope_reference_convention.py:22-35.
    """
    x, angles = np.asarray(x), np.asarray(angles)
    rows, cols = x.shape[0], x.shape[-1]
    lut = angles.shape[0]
    if rows % lut:
        raise ValueError(f"RoPE: angles ({lut} rows) must divide x's {rows} rows")
    xr = _f(x).reshape(lut, -1, cols)
    cos = _f(angles[:, 0::2]).reshape(lut, 1, cols // 2)
    sin = _f(angles[:, 1::2]).reshape(lut, 1, cols // 2)
    out = np.empty_like(xr)
    if two_halves:
        h = cols // 2
        x1, x2 = xr[..., :h], xr[..., h:]
        out[..., :h] = x1 * cos - x2 * sin
        out[..., h:] = x2 * cos + x1 * sin
    else:
        x1, x2 = xr[..., 0::2], xr[..., 1::2]
        out[..., 0::2] = x1 * cos - x2 * sin
        out[..., 1::2] = x2 * cos + x1 * sin
    return out.reshape(x.shape).astype(x.dtype)


def silu(x):
    """``x * sigmoid(x)`` in float32, rounded once -- iron/operators/silu.py:12-22."""
    x = np.asarray(x)
    xf = _f(x)
    return (xf / (1 + np.exp(-xf))).astype(x.dtype)


def add(a, b):
    """``a + b`` (``b`` may be a row) -- iron/operators/elementwise_add.py:11,18."""
    a = np.asarray(a)
    return (_f(a) + _f(b)).astype(a.dtype)


def mul(a, b):
    """``a * b`` (``b`` may be a row) -- iron/operators/elementwise_mul.py:11,18."""
    a = np.asarray(a)
    return (_f(a) * _f(b)).astype(a.dtype)


def axpy(x, y, scalar: float):
    """``scalar * x + y`` -- iron/operators/axpy.py:12-31."""
    x = np.asarray(x)
    return (f32(scalar) * _f(x) + _f(y)).astype(x.dtype)


# ---------------------------------------------------------------------------------------
# Attention


def mha(Q, K, V, *, num_heads, num_kv_heads, causal=True, window=None, scale=None,
        heads_interleaved=False, kv_interleaved=False, q_tokens=None, kv_tokens=None,
        s_q=None, s_kv=None):
    """Attention per head, the queries being the keys' last rows.

    iron/operators/mha.py:1073-1116.  ``q_tokens``/``kv_tokens`` are a bounded call's
    extents (defaults: every row).  Query rows from ``s_q`` on are zeros and keys from
    ``s_kv`` on are masked.
    """
    Q, K, V = np.asarray(Q), np.asarray(K), np.asarray(V)
    if heads_interleaved:
        Q = np.swapaxes(Q, 0, 1)
    if kv_interleaved:
        K, V = (np.swapaxes(t, 0, 1) for t in (K, V))
    d = Q.shape[-1]
    scale = f32(1 / np.sqrt(d)) if scale is None else f32(scale)
    q_tokens = Q.shape[1] if q_tokens is None else q_tokens
    kv_tokens = K.shape[1] if kv_tokens is None else kv_tokens
    groups = num_heads // num_kv_heads
    offset = kv_tokens - q_tokens
    start = offset if causal or window else 0
    s_q = start + q_tokens if s_q is None else int(s_q)
    s_kv = kv_tokens if s_kv is None else int(s_kv)
    K, V = K[:, :s_kv], V[:, :s_kv]
    rows = max(s_q - start, 0)
    q = _f(Q[:, :rows])
    k, v = _f(K), _f(V)
    key = np.arange(k.shape[1])
    out = np.zeros(Q.shape, dtype=Q.dtype)
    step = max(1, 2**24 // max(k.shape[1], 1))
    for first in range(0, rows, step):
        block = slice(first, min(first + step, rows))
        position = offset + np.arange(block.start, block.stop)[:, None]
        masked = np.zeros((len(position), k.shape[1]), dtype=bool)
        if causal or window:
            masked |= key > position + (0 if causal else (window or 0))
        if window:
            masked |= key < position - window
        mask = np.where(masked, -np.inf, 0).astype(f32)
        for h in range(q.shape[0]):
            scores = q[h, block] @ k[h // groups].T * scale + mask
            e = np.exp(scores - scores.max(axis=-1, keepdims=True))
            out[h, block] = (e / e.sum(axis=-1, keepdims=True)) @ v[h // groups]
    if heads_interleaved:
        return np.ascontiguousarray(np.swapaxes(out, 0, 1))
    return out


# ---------------------------------------------------------------------------------------
# Mamba2


def selective_scan(xbc, dt, head, state, *, heads, head_dim, state_size, groups=1, valid=None):
    """The sequential recurrence -- iron/operators/selective_scan.py:367-383.

    Returns ``(y bf16 (rows, inner), final f32 (H, P, N))``.
    """
    H, P, N, G = heads, head_dim, state_size, groups
    inner = H * P
    xbc, dt = np.asarray(xbc, f32), np.asarray(dt, f32)
    rows = xbc.shape[0]
    valid = rows if valid is None else valid
    dt_bias, A, D = np.asarray(head, f32).T
    state = np.array(state, f32)
    y = np.zeros((rows, inner), f32)
    for t in range(valid):
        x = xbc[t, :inner].reshape(H, P)
        B, C = (np.repeat(m.reshape(G, N), H // G, axis=0) for m in np.split(xbc[t, inner:], 2))
        step = np.logaddexp(0, dt[t] + dt_bias)[:, None, None]
        state = np.exp(step * A[:, None, None]) * state
        state += step * x[:, :, None] * B[:, None, :]
        y[t] = (np.einsum("hpn,hn->hp", state, C) + D[:, None] * x).reshape(-1)
    return y.astype(bfloat16), state


def causal_conv1d(x, taps, history=None, bias=None, decode=False):
    """Depth-wise causal filter -- iron/functional.py:147-180 (its recorded steps' references).

    ``y[t] = sum_k taps[k] * x[t - K + 1 + k]`` with the ``K - 1`` rows before ``x`` read
    from ``history`` (zeros if None).  The reference accumulates tap by tap in bf16:
    a prompt chunk records ``y = x_0*taps[0]`` rounded, then ``y = y + bf16(x_k * taps[k])``
    rounded, for k = 1..K-1 (:172-174); a decode step (one unbounded row, ``decode``) starts
    from the newest row, ``y = x*taps[K-1]``, then adds the carried rows oldest first
    (:165-167).  Returns ``(y, new_history)``.
    """
    x, taps = np.asarray(x), np.asarray(taps)
    K, C = taps.shape
    hist = np.zeros((K - 1, C), x.dtype) if history is None else np.asarray(history)
    full = np.concatenate([hist, x], axis=0)
    rows = x.shape[0]
    order = [K - 1, *range(K - 1)] if decode else list(range(K))
    y = mul(full[order[0] : order[0] + rows], taps[order[0]])
    for k in order[1:]:
        y = add(y, mul(full[k : k + rows], taps[k]))
    if bias is not None:
        y = add(y, bias)
    return y, full[rows:]


# ---------------------------------------------------------------------------------------
# Data movement / sampling


def gather_rows(table, ids):
    """``table[ids]`` with ids clipped into range -- iron/common/graph/record.py:465-477."""
    table = np.asarray(table)
    ids = np.clip(np.asarray(ids).astype(np.int64), 0, table.shape[0] - 1)
    return table[ids]


def greedy(logits) -> int:
    """First index of the largest logit -- iron/lm/generation.py:97-99."""
    return int(np.argmax(_f(logits)))
