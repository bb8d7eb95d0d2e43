"""A decoder's modules as graphs (iron/lm/blocks.py): ``Linear``, ``Embedding``, ``RMSNorm``,
``Rope``, ``KVCache``, ``Attention``, ``GatedMLP``, ``DecoderLayer``.

Each ``body`` records operator steps through ``iron_b200.functional`` and handle
arithmetic, so a model's graph is the same sequence of steps the reference records:
per layer RMSNorm, three projections, two RoPE, two cache writes, MHA, o_proj, add,
RMSNorm, gate and up projections, SiLU, multiply, down_proj, add.
"""

from __future__ import annotations

import dataclasses
from functools import partial
from typing import Any

import numpy as np
from ml_dtypes import bfloat16

from .. import functional as F
from ..graph import Graph, param, state, weight
from ..operators.axpy import AXPY
from ..operators.copy import Copy
from ..operators.mha import MHA
from .config import Precision


@dataclasses.dataclass
class Call:
    """What one call of a causal model's body runs (iron/lm/causal.py:40-68)."""

    prompt: bool
    start: Any
    rows: Any
    position: Any
    ids: Any = None
    token: Any = None
    ropes: dict = dataclasses.field(default_factory=dict)


class Linear(Graph):
    """``torch.nn.Linear``: ``x @ weight.T`` (+ ``bias``) at ``precision``."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True, *, precision: Precision):
        self.in_features, self.out_features = in_features, out_features
        self.weight = param(out_features, in_features)
        self.bias = param(out_features) if bias else None
        self.precision = precision

    def body(self, x):
        return F.linear(x, self.weight, self.bias, precision=self.precision)


class Embedding(Graph):
    """``torch.nn.Embedding``: the rows of ``weight`` that ``ids`` name."""

    def __init__(self, num_embeddings: int, embedding_dim: int):
        self.num_embeddings, self.embedding_dim = num_embeddings, embedding_dim
        self.weight = param(num_embeddings, embedding_dim)

    def body(self, ids):
        return Copy.step(weight(self.weight)[ids])


class RMSNorm(Graph):
    """``torch.nn.RMSNorm`` over the last axis, times ``weight``."""

    def __init__(self, normalized_shape, eps: float | None = None):
        n = normalized_shape
        self.normalized_shape = (n,) if isinstance(n, int) else tuple(n)
        self.eps = eps
        self.weight = param(*self.normalized_shape)

    def body(self, x):
        return F.rms_norm(x, self.normalized_shape, self.weight, self.eps)


def residual_add(x, y, residual: float):
    """``x`` plus ``y`` times ``residual``, in ``x``'s shape."""
    y = y if y.shape == x.shape else y.reshape(x.shape)
    if residual == 1:
        return x + y
    n = x.elements
    return AXPY.step(y.reshape(n), x.reshape(n), scalar_factor=residual).reshape(x.shape)


class Rope(Graph):
    """A decoder's RoPE table, one bf16 row per position; a call copies its rows once for all layers."""

    def __init__(self, c):
        self.table = weight(c.angles().astype(bfloat16))
        self.chunk, self.width = c.prefill_chunk, c.rope_width

    def rows(self, call: Call):
        if call.prompt:
            k = Copy.step(self.table[call.start : call.start + self.chunk][: call.rows])
        else:
            k = Copy.step(self.table[call.position]).reshape(1, self.width)
        return k, k


class KVCache(Graph):
    """A layer's keys and values ``(max_seq_len, groups, head_dim)`` and causal attention over them."""

    def __init__(self, c, window: int | None = None):
        G, D = c.num_key_value_heads, c.head_dim
        self.chunk, self.window = c.prefill_chunk, window
        self.keys, self.values = state((c.max_seq_len, G, D)), state((c.max_seq_len, G, D))

    def attend(self, call: Call, q, k, v, scale: float | None = None):
        C, (_, G, D), (n, H, _) = self.chunk, self.keys.shape, q.shape
        for x, cache in ((k, self.keys), (v, self.values)):
            if call.prompt:
                cache[call.start : call.start + C][: call.rows] = x
            else:
                cache[call.position] = x.reshape(G, D)
        keys, values = (x[: call.position + 1] for x in (self.keys, self.values))
        o = MHA.step(q, keys, values, heads_interleaved=True, kv_interleaved=True, window=self.window,
                     scale=scale, seq_len=n if n == 1 else None)
        return o.reshape(n, H * D)


class Attention(Graph):
    """Self-attention of one decoder layer: q, k, v project, RoPE rotates, the cache attends."""

    def __init__(self, c, i: int, o_bias: bool = False):
        H, G, D, E = c.num_attention_heads, c.num_key_value_heads, c.head_dim, c.hidden_size
        self.heads, self.groups, self.head_dim = H, G, D
        linear = partial(Linear, bias=c.attention_bias, precision=c.precision)
        self.q_proj, self.k_proj, self.v_proj = linear(E, H * D), linear(E, G * D), linear(E, G * D)
        self.o_proj = Linear(H * D, E, bias=o_bias, precision=c.precision)
        self.scaling: float | None = None   # the logits' scale; None is 1 / sqrt(head_dim)

    def body(self, x, cache: KVCache, call: Call, angles=None):
        n, H, G, D = x.shape[0], self.heads, self.groups, self.head_dim
        q, k, v = (p(x) for p in (self.q_proj, self.k_proj, self.v_proj))
        q, k, v = q.reshape(n * H, D), k.reshape(n * G, D), v.reshape(n * G, D)
        if angles is not None:
            q, k = F.rope(q, angles[0]), F.rope(k, angles[1])
        o = cache.attend(call, q.reshape(n, H, D), k.reshape(n, G, D), v.reshape(n, G, D), scale=self.scaling)
        return self.o_proj(o)


class GatedMLP(Graph):
    """``down_proj(silu(gate_proj(x)) * up_proj(x))``."""

    def __init__(self, c):
        E, M = c.hidden_size, c.intermediate_size
        linear = partial(Linear, bias=c.mlp_bias, precision=c.precision)
        self.gate_proj, self.up_proj, self.down_proj = linear(E, M), linear(E, M), linear(M, E)

    def body(self, x):
        return self.down_proj(F.silu(self.gate_proj(x)) * self.up_proj(x))


class DecoderLayer(Graph):
    """Layer ``i`` of a pre-norm decoder."""

    def __init__(self, c, i: int):
        self.input_layernorm = RMSNorm(c.hidden_size, c.eps)
        self.self_attn = Attention(c, i, o_bias=c.attention_bias)
        self.post_attention_layernorm = RMSNorm(c.hidden_size, c.eps)
        self.mlp = GatedMLP(c)
        self.cache = KVCache(c, c.window)
        self.rope = None
        self.residual_multiplier = 1.0

    def body(self, x, call: Call):
        x = residual_add(x, self.mix(self.input_layernorm(x), call), self.residual_multiplier)
        return residual_add(x, self.mlp(self.post_attention_layernorm(x)), self.residual_multiplier)

    def mix(self, h, call: Call):
        """Attend the normed rows ``h`` over the layer's cache (iron/lm/blocks.py:729-733); a
        layer that mixes positions another way (a Mamba2 mixer) overrides it."""
        angles = None if self.rope is None else call.ropes[self.rope]
        return self.self_attn(h, self.cache, call, angles)
