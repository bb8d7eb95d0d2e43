"""CPU oracle for the model path: numpy decoders (Llama, biased Llama, Granite, the Granite 4.0-H
hybrid with Mamba2 mixers) and the float32 transformers judge.

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


# ---------------------------------------------------------------------------------------
# Granite, biased Llama and the Granite 4.0-H hybrid (Mamba2 mixers): the other toys the
# reference records goldens for


@dataclasses.dataclass(frozen=True)
class DecoderShape(LlamaShape):
    """``LlamaShape`` plus what the reference's other decoders read from their configs:
    projection biases (iron/lm/config.py ``attention_bias``), Granite's four scalars
    (iron/applications/granite/model.py:32-43) and the hybrid's Mamba2 mixer shape
    (iron/applications/granite_hybrid/model.py:37-86).  ``rope_theta`` None is no RoPE."""

    rope_theta: float | None = 500000.0
    attention_bias: bool = False
    attention_multiplier: float | None = None
    residual_multiplier: float = 1.0
    embedding_multiplier: float = 1.0
    logits_scaling: float = 1.0
    layer_types: tuple[str, ...] | None = None
    shared_intermediate_size: int | None = None
    mamba_n_heads: int = 0
    mamba_d_head: int = 0
    mamba_d_state: int = 0
    mamba_n_groups: int = 1
    mamba_d_conv: int = 4

    def attends(self, i: int) -> bool:
        return self.layer_types is None or self.layer_types[i] in ("attention", "full_attention")

    @property
    def d_inner(self) -> int:
        return self.mamba_n_heads * self.mamba_d_head

    @property
    def conv_channels(self) -> int:
        return self.d_inner + 2 * self.mamba_n_groups * self.mamba_d_state


#: tests/applications/llama/reference/test.py:23-26: ``SMALL`` with a bias on q, k, v and o.
BIASED = DecoderShape(
    vocab_size=1024, hidden_size=512, num_hidden_layers=2, num_attention_heads=16,
    num_key_value_heads=4, head_dim=64, intermediate_size=2048, max_seq_len=256,
    prefill_chunk=256, attention_bias=True,
)

#: tests/applications/granite/reference/test.py:18-33.
GRANITE_TOY = DecoderShape(
    vocab_size=1024, hidden_size=512, num_hidden_layers=2, num_attention_heads=8,
    num_key_value_heads=2, head_dim=64, intermediate_size=1024, rope_theta=10000.0,
    max_seq_len=256, prefill_chunk=256, eps=1e-6, tie_word_embeddings=False,
    attention_multiplier=0.0625, residual_multiplier=0.22, embedding_multiplier=12.0,
    logits_scaling=8.0,
)

#: tests/applications/granite_hybrid/reference/test.py:28-51: three Mamba2 layers of two
#: groups, one attention layer without RoPE, the shared gated MLP, an untied head.
HYBRID_TOY = DecoderShape(
    vocab_size=1024, hidden_size=512, num_hidden_layers=4, num_attention_heads=8,
    num_key_value_heads=2, head_dim=64, intermediate_size=256, rope_theta=None,
    max_seq_len=256, prefill_chunk=64, eps=1e-6, tie_word_embeddings=False,
    attention_multiplier=0.0625, residual_multiplier=0.22, embedding_multiplier=12.0,
    logits_scaling=8.0, layer_types=("mamba", "attention", "mamba", "mamba"),
    shared_intermediate_size=512, mamba_n_heads=16, mamba_d_head=64, mamba_d_state=64,
    mamba_n_groups=2,
)


def decoder_shapes(c: DecoderShape) -> dict[str, tuple[int, ...]]:
    """Checkpoint names and shapes in the reference's draw order: Llama's table, then the
    biases (tests/applications/llama/reference/test.py:29-41) or the untied head
    (tests/applications/granite/reference/test.py:41-43); the hybrid's own table
    (tests/applications/granite_hybrid/reference/test.py:88-127)."""
    E, V = c.hidden_size, c.vocab_size
    Q, KV = c.num_attention_heads * c.head_dim, c.num_key_value_heads * c.head_dim
    if c.layer_types is None:
        out = llama_shapes(c)
        if c.attention_bias:
            for i in range(c.num_hidden_layers):
                a = f"model.layers.{i}.self_attn"
                out |= {f"{a}.q_proj.bias": (Q,), f"{a}.k_proj.bias": (KV,), f"{a}.v_proj.bias": (KV,),
                        f"{a}.o_proj.bias": (E,)}
        if not c.tie_word_embeddings:
            out |= {"lm_head.weight": (V, E)}
        return out
    S, H, N = c.shared_intermediate_size, c.mamba_n_heads, c.mamba_d_state
    out = {"model.embed_tokens.weight": (V, E), "model.norm.weight": (E,), "lm_head.weight": (V, E)}
    for i in range(c.num_hidden_layers):
        p = f"model.layers.{i}"
        out |= {f"{p}.input_layernorm.weight": (E,), f"{p}.post_attention_layernorm.weight": (E,),
                f"{p}.shared_mlp.input_linear.weight": (2 * S, E),
                f"{p}.shared_mlp.output_linear.weight": (E, S)}
        if c.attends(i):
            out |= {f"{p}.self_attn.q_proj.weight": (Q, E), f"{p}.self_attn.k_proj.weight": (KV, E),
                    f"{p}.self_attn.v_proj.weight": (KV, E), f"{p}.self_attn.o_proj.weight": (E, Q)}
        else:
            m = f"{p}.mamba"
            out |= {f"{m}.in_proj.weight": (c.d_inner + c.conv_channels + H, E),
                    f"{m}.conv1d.weight": (c.conv_channels, 1, c.mamba_d_conv),
                    f"{m}.conv1d.bias": (c.conv_channels,), f"{m}.dt_bias": (H,), f"{m}.A_log": (H,),
                    f"{m}.D": (H,), f"{m}.norm.weight": (c.d_inner,), f"{m}.out_proj.weight": (E, c.d_inner)}
    return out


def hybrid_redraw(c: DecoderShape, weights: dict[str, np.ndarray]) -> dict[str, np.ndarray]:
    """The hybrid toy's weights after the reference's own redraw, in place
    (tests/applications/granite_hybrid/reference/test.py:62-71): decays and time steps as
    Mamba2 initialises them, the convolution's bias ten times the shared draw's."""
    rng = np.random.default_rng(0)
    H = c.mamba_n_heads
    for i in range(c.num_hidden_layers):
        if c.attends(i):
            continue
        m = f"model.layers.{i}.mamba"
        weights[f"{m}.A_log"][:] = np.log(rng.uniform(1, 16, H))
        dt = np.exp(rng.uniform(np.log(1e-3), np.log(1e-1), H))
        weights[f"{m}.dt_bias"][:] = dt + np.log(-np.expm1(-dt))
        weights[f"{m}.conv1d.bias"][:] *= 10
    return weights


def mamba_mixer(h, w, prefix, conv_state, ssm_state, *, heads, head_dim, state_size, groups=1, kernel=4,
                eps=1e-5):
    """One Mamba2 mixer over the rows ``h`` of one sequence, operator by operator as
    iron/applications/granite_hybrid/model.py:120-137 records it: three projections on row
    slices of ``in_proj``, the causal convolution plus its bias, SiLU, the scan, the product
    with SiLU of the gate, RMSNorm over ``d_inner``, ``out_proj``.  ``conv_state`` is the
    ``kernel - 1`` rows before ``h``, ``ssm_state`` the scan's float32 state; returns
    ``(out, conv_state, ssm_state)`` after the rows."""
    lin = lambda x, W: (np.asarray(x, np.float32) @ np.asarray(W, np.float32).T).astype(bfloat16)
    d_inner = heads * head_dim
    C = d_inner + 2 * groups * state_size
    W = w[prefix + "in_proj.weight"]
    gate, xbc, dt = (lin(h, part) for part in (W[:d_inner], W[d_inner : d_inner + C], W[d_inner + C :]))
    taps = np.ascontiguousarray(np.asarray(w[prefix + "conv1d.weight"]).reshape(C, kernel).T)
    # a call of one row is a decode step, which sums the taps in its own order
    conv, conv_state = ops.causal_conv1d(xbc, taps, conv_state, w[prefix + "conv1d.bias"], decode=h.shape[0] == 1)
    A = -np.exp(np.asarray(w[prefix + "A_log"], np.float32))
    head = np.stack([np.asarray(w[prefix + "dt_bias"], np.float32), A, np.asarray(w[prefix + "D"], np.float32)],
                    1).astype(np.float32)
    y, ssm_state = ops.selective_scan(ops.silu(conv), dt, head, ssm_state, heads=heads, head_dim=head_dim,
                                      state_size=state_size, groups=groups)
    y = ops.rms_norm(ops.mul(y, ops.silu(gate)), w[prefix + "norm.weight"], eps)
    return lin(y, w[prefix + "out_proj.weight"]), conv_state, ssm_state


class NumpyDecoder:
    """The reference's host graph for its other decoders, operator by operator in bf16:
    Llama's layer with optional biases and Granite's scalars
    (iron/applications/granite/model.py:46-93: attention scale, AXPY residuals, the embedding
    row product, the logits' divisor folded into the final norm's weight), and the hybrid's
    layer (iron/applications/granite_hybrid/model.py:87-176): a Mamba2 mixer or attention,
    then the shared gated MLP.  The mixer's states -- the convolution's last ``K - 1`` rows
    and the scan's float32 state -- carry from call to call as the reference's
    ``Checkpoints`` do (iron/lm/causal.py:71-121)."""

    def __init__(self, config: DecoderShape, weights: dict[str, np.ndarray]):
        self.c, self.w = c, w = config, weights
        self.angles = None if c.rope_theta is None else c.angles().astype(bfloat16)
        G, D, L = c.num_key_value_heads, c.head_dim, c.num_hidden_layers
        self.keys = [np.zeros((c.max_seq_len, G, D), bfloat16) for _ in range(L)]
        self.values = [np.zeros((c.max_seq_len, G, D), bfloat16) for _ in range(L)]
        K = c.mamba_d_conv
        self.conv = [np.zeros((K - 1, c.conv_channels), bfloat16) for _ in range(L)]
        self.ssm = [np.zeros((c.mamba_n_heads, c.mamba_d_head, c.mamba_d_state), np.float32) for _ in range(L)]
        self.embed_scale = np.full(c.hidden_size, c.embedding_multiplier, bfloat16)
        norm = np.asarray(w["model.norm.weight"])
        # the reference divides in bf16 (iron/applications/granite/model.py:81-83)
        self.final_norm = norm if c.logits_scaling == 1 else (norm / bfloat16(c.logits_scaling)).astype(bfloat16)

    def _linear(self, x, W, bias=None):
        y = (np.asarray(x, np.float32) @ np.asarray(W, np.float32).T).astype(bfloat16)
        return y if bias is None else ops.add(y, np.broadcast_to(bias, y.shape))

    def _residual(self, x, y):
        r = self.c.residual_multiplier
        return ops.add(x, y) if r == 1 else ops.axpy(y, x, r)

    def _attention(self, i, h, start):
        c, w = self.c, self.w
        H, G, D = c.num_attention_heads, c.num_key_value_heads, c.head_dim
        n, a = h.shape[0], f"model.layers.{i}.self_attn"
        bias = (lambda p: w[f"{a}.{p}.bias"]) if c.attention_bias else (lambda p: None)
        q = self._linear(h, w[f"{a}.q_proj.weight"], bias("q_proj")).reshape(n * H, D)
        k = self._linear(h, w[f"{a}.k_proj.weight"], bias("k_proj")).reshape(n * G, D)
        v = self._linear(h, w[f"{a}.v_proj.weight"], bias("v_proj")).reshape(n, G, D)
        if self.angles is not None:
            ang = self.angles[start : start + n]
            q, k = ops.rope(q, ang), ops.rope(k, ang)
        self.keys[i][start : start + n] = k.reshape(n, G, D)
        self.values[i][start : start + n] = v
        kv = start + n
        o = ops.mha(q.reshape(n, H, D), self.keys[i][:kv], self.values[i][:kv], num_heads=H, num_kv_heads=G,
                    heads_interleaved=True, kv_interleaved=True, scale=c.attention_multiplier).reshape(n, H * D)
        return self._linear(o, w[f"{a}.o_proj.weight"], bias("o_proj"))

    def _mamba(self, i, h):
        c = self.c
        out, self.conv[i], self.ssm[i] = mamba_mixer(
            h, self.w, f"model.layers.{i}.mamba.", self.conv[i], self.ssm[i], heads=c.mamba_n_heads,
            head_dim=c.mamba_d_head, state_size=c.mamba_d_state, groups=c.mamba_n_groups, kernel=c.mamba_d_conv,
            eps=c.eps)
        return out

    def _mlp(self, i, h):
        c, w, p = self.c, self.w, f"model.layers.{i}"
        if c.layer_types is None:
            gate = self._linear(h, w[f"{p}.mlp.gate_proj.weight"])
            up = self._linear(h, w[f"{p}.mlp.up_proj.weight"])
            return self._linear(ops.mul(ops.silu(gate), up), w[f"{p}.mlp.down_proj.weight"])
        S, W = c.shared_intermediate_size, w[f"{p}.shared_mlp.input_linear.weight"]
        gate, up = self._linear(h, W[:S]), self._linear(h, W[S:])
        return self._linear(ops.mul(ops.silu(gate), up), w[f"{p}.shared_mlp.output_linear.weight"])

    def forward(self, tokens, start: int):
        """Run ``tokens`` at positions ``start...`` (in order: the mixers' states carry on);
        logits of the last row, bf16."""
        c, w = self.c, self.w
        tokens = np.asarray(tokens).reshape(-1)
        n = len(tokens)
        x = ops.gather_rows(w["model.embed_tokens.weight"], tokens)
        if c.embedding_multiplier != 1:
            x = ops.mul(x, np.broadcast_to(self.embed_scale, x.shape))
        for i in range(c.num_hidden_layers):
            p = f"model.layers.{i}"
            h = ops.rms_norm(x, w[f"{p}.input_layernorm.weight"], c.eps)
            x = self._residual(x, self._attention(i, h, start) if c.attends(i) else self._mamba(i, h))
            h = ops.rms_norm(x, w[f"{p}.post_attention_layernorm.weight"], c.eps)
            x = self._residual(x, self._mlp(i, h))
        last = ops.rms_norm(x[n - 1 : n], self.final_norm, c.eps)
        head = w.get("lm_head.weight", w["model.embed_tokens.weight"])
        return self._linear(last, head).reshape(-1)

    def logits(self, tokens):
        """Logits after the last of ``tokens`` from empty states, in prompt chunks."""
        tokens = np.asarray(tokens).reshape(-1)
        C, out = self.c.prefill_chunk, None
        for s in range(0, len(tokens), C):
            out = self.forward(tokens[s : s + C], s)
        return out


def hf_decoder(model_type: str, c: DecoderShape, weights: dict[str, np.ndarray]):
    """transformers' ``model_type`` ("llama", "granite", "granitemoehybrid") in float32 on
    ``weights``, its config the fields ``c`` would write to a ``config.json``
    (iron/lm/golden.py:193-224; the hybrid adds ``mamba_expand`` as
    tests/applications/granite_hybrid/reference/test.py:83 does)."""
    import tempfile

    import torch
    import transformers
    from safetensors.torch import save_file

    cfg = dict(vocab_size=c.vocab_size, hidden_size=c.hidden_size, num_hidden_layers=c.num_hidden_layers,
               num_attention_heads=c.num_attention_heads, num_key_value_heads=c.num_key_value_heads,
               head_dim=c.head_dim, intermediate_size=c.intermediate_size,
               max_position_embeddings=c.max_seq_len, rms_norm_eps=c.eps, hidden_act="silu",
               tie_word_embeddings=c.tie_word_embeddings, attention_bias=c.attention_bias, mlp_bias=False)
    if c.rope_theta is not None:
        cfg["rope_theta"] = c.rope_theta
    if c.attention_multiplier is not None:
        cfg |= dict(attention_multiplier=c.attention_multiplier, residual_multiplier=c.residual_multiplier,
                    embedding_multiplier=c.embedding_multiplier, logits_scaling=c.logits_scaling)
    if c.layer_types is not None:
        cfg |= dict(layer_types=list(c.layer_types), position_embedding_type="nope",
                    shared_intermediate_size=c.shared_intermediate_size, num_local_experts=0,
                    num_experts_per_tok=2, mamba_n_heads=c.mamba_n_heads, mamba_d_head=c.mamba_d_head,
                    mamba_d_state=c.mamba_d_state, mamba_n_groups=c.mamba_n_groups,
                    mamba_d_conv=c.mamba_d_conv, mamba_expand=2, rope_theta=10000.0)
    hf = transformers.AutoConfig.for_model(model_type, **cfg)
    with tempfile.TemporaryDirectory() as directory:
        hf.save_pretrained(directory)
        save_file({k: torch.from_numpy(np.asarray(v).astype(np.float32)) for k, v in weights.items()},
                  f"{directory}/model.safetensors")
        model, info = transformers.AutoModelForCausalLM.from_pretrained(
            directory, dtype=torch.float32, output_loading_info=True)
    if info["missing_keys"] or info["unexpected_keys"]:
        raise ValueError(f"weights lack {sorted(info['missing_keys'])} and hold {sorted(info['unexpected_keys'])}")
    return model.eval()
