"""CPU oracle for the model path: a numpy Llama decoder and the float32 transformers judge.

TEST INFRASTRUCTURE ONLY (see ``oracle/ops.py``).

``NumpyLlama`` replays what the reference's ``Graph.reference`` does for the Llama graph
(iron/common/graph/record.py:340-448 running every recorded step's ``reference()``):
bf16 tensors, float32 arithmetic, one rounding per operator, in the order
``iron/lm/blocks.py:627-648`` (attention), ``:472-502`` (KV cache), ``:697-699`` (gated MLP),
``:723-728`` (layer) and ``iron/lm/causal.py:271-332`` (embedding, layers, final norm, head)
record them.  ``hf_llama`` builds the float32 Hugging Face model the reference judges a
model by (iron/lm/golden.py:193-238).
"""

from __future__ import annotations

import dataclasses
import hashlib
import math

import numpy as np
from ml_dtypes import bfloat16

from . import ops


# ---------------------------------------------------------------------------------------
# RoPE table


def rope_angles(head_dim, context_length, rope_theta=500000.0, scaling=None):
    """``(context_length, head_dim)`` float32, cos at even and sin at odd columns.

    iron/lm/config.py:23-42: float64 trigonometry of (f32 position x f32 inv_freq),
    rounded once.
    """
    exponents = np.arange(0, head_dim, 2, dtype=np.float32) / np.float32(head_dim)
    inv_freq = 1.0 / np.power(rope_theta, exponents.astype(np.float64))
    if scaling is not None:
        inv_freq = scaling(inv_freq)
    inv_freq = inv_freq.astype(np.float32)
    freqs = np.outer(np.arange(context_length, dtype=np.float32), inv_freq)
    angles = np.empty((context_length, head_dim), dtype=np.float32)
    angles[:, ::2] = np.cos(freqs.astype(np.float64))
    angles[:, 1::2] = np.sin(freqs.astype(np.float64))
    return angles


@dataclasses.dataclass(frozen=True)
class Llama3RopeScaling:
    """Llama 3's frequency scaling -- iron/applications/llama/model.py:25-55."""

    factor: float
    low_freq_factor: float
    high_freq_factor: float
    original_max_position_embeddings: int
    rope_type: str = "llama3"

    def __call__(self, inv_freq):
        original = self.original_max_position_embeddings
        wavelen = 2 * np.pi / inv_freq
        smooth = (original / wavelen - self.low_freq_factor) / (
            self.high_freq_factor - self.low_freq_factor
        )
        between = (1 - smooth) * inv_freq / self.factor + smooth * inv_freq
        return np.where(
            wavelen < original / self.high_freq_factor,
            inv_freq,
            np.where(wavelen > original / self.low_freq_factor, inv_freq / self.factor, between),
        )


# ---------------------------------------------------------------------------------------
# Config and weights


@dataclasses.dataclass(frozen=True)
class LlamaShape:
    """The fields of the reference's ``LlamaConfig`` the decoder path reads."""

    vocab_size: int = 128256
    hidden_size: int = 2048
    num_hidden_layers: int = 16
    num_attention_heads: int = 32
    num_key_value_heads: int = 8
    head_dim: int = 64
    intermediate_size: int = 8192
    rope_theta: float = 500000.0
    max_seq_len: int = 2304
    eps: float = 1e-5
    prefill_chunk: int = 2048
    rope_scaling: Llama3RopeScaling | None = None
    tie_word_embeddings: bool = True

    def angles(self):
        return rope_angles(self.head_dim, self.max_seq_len, self.rope_theta, self.rope_scaling)


#: iron/tests/support/llama_model.py:56-68 (``SMALL``) and
#: iron/tests/common/test_llama_reference.py:52-60 (``SCALED``): the toy the goldens use.
SMALL = LlamaShape(
    vocab_size=1024, hidden_size=512, num_hidden_layers=2, num_attention_heads=16,
    num_key_value_heads=4, head_dim=64, intermediate_size=2048, max_seq_len=256,
    prefill_chunk=256, rope_scaling=None,
)
SCALED = dataclasses.replace(
    SMALL,
    rope_scaling=Llama3RopeScaling(
        factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
        original_max_position_embeddings=64,
    ),
)


def llama_shapes(c: LlamaShape) -> dict[str, tuple[int, ...]]:
    """Checkpoint tensor names and shapes in draw order -- iron/tests/support/llama_model.py:76-98."""
    E, F, V = c.hidden_size, c.intermediate_size, c.vocab_size
    Q, KV = c.num_attention_heads * c.head_dim, c.num_key_value_heads * c.head_dim
    out = {"model.embed_tokens.weight": (V, E), "model.norm.weight": (E,)}
    for i in range(c.num_hidden_layers):
        layer = f"model.layers.{i}"
        out |= {
            f"{layer}.input_layernorm.weight": (E,),
            f"{layer}.self_attn.q_proj.weight": (Q, E),
            f"{layer}.self_attn.k_proj.weight": (KV, E),
            f"{layer}.self_attn.v_proj.weight": (KV, E),
            f"{layer}.self_attn.o_proj.weight": (E, Q),
            f"{layer}.post_attention_layernorm.weight": (E,),
            f"{layer}.mlp.gate_proj.weight": (F, E),
            f"{layer}.mlp.up_proj.weight": (F, E),
            f"{layer}.mlp.down_proj.weight": (E, F),
        }
    return out


def filled_random(named: dict[str, tuple[int, ...]], seed: int = 0, dtype=bfloat16):
    """The reference's ``filled("random")`` draw -- iron/common/graph/fill.py:24-33.

    One ``default_rng(seed)`` stream in name order: matrices ``N(0,1)/sqrt(in)``, vectors
    ``1 + N(0,1)/10`` (a bias without the one), drawn float32 then cast.
    """
    rng = np.random.default_rng(seed)
    out = {}
    for n, shape in named.items():
        x = rng.standard_normal(shape, dtype=np.float32)
        if len(shape) >= 2:
            out[n] = (x / np.sqrt(math.prod(shape[1:]))).astype(dtype)
        else:
            out[n] = np.asarray(x / 10 + (not n.endswith("bias")), dtype)
    return out


def filled_normal(named: dict[str, tuple[int, ...]], seed: int, std: float = 0.02, dtype=bfloat16):
    """The benchmark draw: matrices ``N(0, std)``, norm weights one."""
    rng = np.random.default_rng(seed)
    out = {}
    for n, shape in named.items():
        if len(shape) >= 2:
            out[n] = (rng.standard_normal(shape, dtype=np.float32) * np.float32(std)).astype(dtype)
        else:
            out[n] = np.ones(shape, dtype)
    return out


def golden_key(tokens) -> str:
    """A golden row's name: sha256 of the int64 token bytes -- iron/lm/golden.py:88-92."""
    return hashlib.sha256(np.asarray(tokens, np.int64).tobytes()).hexdigest()[:16]


# ---------------------------------------------------------------------------------------
# The bf16 numpy decoder


class NumpyLlama:
    """Llama decoder on ``weights`` (checkpoint names), every operator rounding to bf16."""

    def __init__(self, config: LlamaShape, weights: dict[str, np.ndarray]):
        self.c, self.w = config, weights
        c = config
        self.angles = c.angles().astype(bfloat16)
        G, D = c.num_key_value_heads, c.head_dim
        self.keys = [np.zeros((c.max_seq_len, G, D), bfloat16) for _ in range(c.num_hidden_layers)]
        self.values = [np.zeros((c.max_seq_len, G, D), bfloat16) for _ in range(c.num_hidden_layers)]
        self.held = 0  # positions the caches hold

    def _linear(self, x, name):
        # one row -> GEMV, several -> ProjectionGEMM; both bf16(f32 x @ W.T)
        W = self.w[name]
        return (x.astype(np.float32) @ W.astype(np.float32).T).astype(bfloat16)

    def forward(self, tokens, start: int):
        """Run ``tokens`` at positions ``start...`` over the caches; logits of the last row (bf16)."""
        c = self.c
        H, G, D = c.num_attention_heads, c.num_key_value_heads, c.head_dim
        tokens = np.asarray(tokens).reshape(-1)
        n = len(tokens)
        x = ops.gather_rows(self.w["model.embed_tokens.weight"], tokens)
        ang = self.angles[start : start + n]
        for i in range(c.num_hidden_layers):
            L = f"model.layers.{i}"
            h = ops.rms_norm(x, self.w[f"{L}.input_layernorm.weight"], c.eps)
            q = self._linear(h, f"{L}.self_attn.q_proj.weight").reshape(n * H, D)
            k = self._linear(h, f"{L}.self_attn.k_proj.weight").reshape(n * G, D)
            v = self._linear(h, f"{L}.self_attn.v_proj.weight").reshape(n, G, D)
            q = ops.rope(q, ang).reshape(n, H, D)
            k = ops.rope(k, ang).reshape(n, G, D)
            self.keys[i][start : start + n] = k
            self.values[i][start : start + n] = v
            kv = start + n
            o = ops.mha(
                q, self.keys[i][:kv], self.values[i][:kv], num_heads=H, num_kv_heads=G,
                heads_interleaved=True, kv_interleaved=True,
            ).reshape(n, H * D)
            x = ops.add(x, self._linear(o, f"{L}.self_attn.o_proj.weight"))
            h = ops.rms_norm(x, self.w[f"{L}.post_attention_layernorm.weight"], c.eps)
            gate = self._linear(h, f"{L}.mlp.gate_proj.weight")
            up = self._linear(h, f"{L}.mlp.up_proj.weight")
            x = ops.add(x, self._linear(ops.mul(ops.silu(gate), up), f"{L}.mlp.down_proj.weight"))
        last = ops.rms_norm(x[n - 1 : n], self.w["model.norm.weight"], c.eps)
        head = self.w.get("lm_head.weight", self.w["model.embed_tokens.weight"])
        self.held = start + n
        return (last.astype(np.float32) @ head.astype(np.float32).T).astype(bfloat16).reshape(-1)

    def logits(self, tokens):
        """Logits after the last of ``tokens`` from an empty cache, in prompt chunks."""
        tokens = np.asarray(tokens).reshape(-1)
        C, out = self.c.prefill_chunk, None
        for s in range(0, len(tokens), C):
            out = self.forward(tokens[s : s + C], s)
        return out


# ---------------------------------------------------------------------------------------
# The float32 judge


def hf_llama(c: LlamaShape, weights: dict[str, np.ndarray]):
    """transformers' Llama in float32 on ``weights`` -- iron/lm/golden.py:193-224.

    Built in memory (the reference round-trips through a safetensors file; the state
    dict is the same).  Returns the ``torch.nn.Module`` in eval mode.
    """
    import torch
    import transformers

    rope = None
    if c.rope_scaling is not None:
        rope = dataclasses.asdict(c.rope_scaling)
    cfg = transformers.LlamaConfig(
        vocab_size=c.vocab_size, hidden_size=c.hidden_size,
        num_hidden_layers=c.num_hidden_layers, num_attention_heads=c.num_attention_heads,
        num_key_value_heads=c.num_key_value_heads, head_dim=c.head_dim,
        intermediate_size=c.intermediate_size, rope_theta=c.rope_theta,
        max_position_embeddings=c.max_seq_len, rms_norm_eps=c.eps, rope_scaling=rope,
        tie_word_embeddings=c.tie_word_embeddings, attention_bias=False, mlp_bias=False,
        hidden_act="silu",
    )
    model = transformers.LlamaForCausalLM(cfg).to(torch.float32)
    state = {k: torch.from_numpy(np.asarray(v).astype(np.float32)) for k, v in weights.items()}
    missing, unexpected = model.load_state_dict(state, strict=False)
    missing = [m for m in missing if not (c.tie_word_embeddings and m == "lm_head.weight")]
    if missing or unexpected:
        raise ValueError(f"weights lack {missing} and hold {unexpected}")
    if c.tie_word_embeddings:
        model.tie_weights()
    return model.eval()


def hf_logits(model, tokens) -> np.ndarray:
    """Float32 logits after the last of ``tokens`` (``use_cache=False``) -- golden.py:226-238."""
    import torch

    with torch.no_grad():
        out = model(torch.tensor([list(map(int, tokens))]), use_cache=False)
    return out.logits[0, -1].numpy()
