"""Llama 3 on the shared decoder (iron/applications/llama/model.py:25-99)."""

from __future__ import annotations

import dataclasses
from pathlib import Path

import numpy as np

from ...lm.config import DecoderConfig, Precision, not_json


@dataclasses.dataclass(frozen=True)
class Llama3RopeScaling:
    """Llama 3's RoPE frequency scaling (``"rope_type": "llama3"``).

    Wavelengths shorter than ``original / high_freq_factor`` are kept, longer than
    ``original / low_freq_factor`` are stretched by ``factor``, and the band between is
    blended linearly in ``original / wavelength``.
    """

    factor: float
    low_freq_factor: float
    high_freq_factor: float
    original_max_position_embeddings: int
    rope_type: str = "llama3"

    def __call__(self, inv_freq: np.ndarray) -> np.ndarray:
        n = self.original_max_position_embeddings
        wavelength = 2 * np.pi / inv_freq
        blend = (n / wavelength - self.low_freq_factor) / (self.high_freq_factor - self.low_freq_factor)
        mixed = (1 - blend) * inv_freq / self.factor + blend * inv_freq
        stretched = np.where(wavelength > n / self.low_freq_factor, inv_freq / self.factor, mixed)
        return np.where(wavelength < n / self.high_freq_factor, inv_freq, stretched)

    @classmethod
    def from_dict(cls, data: dict) -> "Llama3RopeScaling":
        if data.get("rope_type") != "llama3":
            raise ValueError(f"rope_scaling {data}: no RoPE table here builds it")
        return cls(**data)


@dataclasses.dataclass(frozen=True)
class LlamaConfig(DecoderConfig):
    """``DecoderConfig`` with Llama 3's own ``rope_scaling`` and a default precision."""

    rope_scaling: Llama3RopeScaling | None = dataclasses.field(
        default=None, metadata={"convert": Llama3RopeScaling.from_dict})
    precision: Precision = not_json(Precision.MEDIUM, kw_only=True)

    @classmethod
    def from_json(cls, data: dict, source="config.json") -> "LlamaConfig":
        config = super().from_json(data, source)
        if config.hidden_size < 3072:
            return config
        return dataclasses.replace(config, precision=Precision.HIGH)


#: Llama 3.2 1B's shape (iron/tests/support/llama_model.py:36-53).
LLAMA_1B = LlamaConfig(
    vocab_size=128256, hidden_size=2048, num_hidden_layers=16, num_attention_heads=32,
    num_key_value_heads=8, head_dim=64, intermediate_size=8192, rope_theta=500000.0,
    max_seq_len=131072, eps=1e-5,
    rope_scaling=Llama3RopeScaling(32.0, 1.0, 4.0, 8192),
)

#: Llama 3.2 3B's shape.
LLAMA_3B = LlamaConfig(
    vocab_size=128256, hidden_size=3072, num_hidden_layers=28, num_attention_heads=24,
    num_key_value_heads=8, head_dim=128, intermediate_size=8192, rope_theta=500000.0,
    max_seq_len=131072, eps=1e-5, precision=Precision.HIGH,
    rope_scaling=Llama3RopeScaling(32.0, 1.0, 4.0, 8192),
)


#: tunables by operator shape, one file per device (``b200.json``), as the reference keeps its
#: ``profiles/npu2.json`` beside the model (iron/applications/llama/model.py:97)
PROFILES = Path(__file__).with_name("profiles")


def checkpoint_shapes(c: DecoderConfig) -> dict[str, tuple[int, ...]]:
    """A Llama checkpoint's tensor names and shapes for ``c``, in the order the reference's
    random fill draws them (iron/tests/support/llama_model.py:76-98); ``lm_head.weight`` only
    when the head is not tied to the embedding."""
    E, F, V = c.hidden_size, c.intermediate_size, c.vocab_size
    Q, KV = c.num_attention_heads * c.head_dim, c.num_key_value_heads * c.head_dim
    out: dict[str, tuple[int, ...]] = {"model.embed_tokens.weight": (V, E), "model.norm.weight": (E,)}
    for i in range(c.num_hidden_layers):
        p = f"model.layers.{i}"
        out[f"{p}.input_layernorm.weight"] = (E,)
        out[f"{p}.self_attn.q_proj.weight"] = (Q, E)
        out[f"{p}.self_attn.k_proj.weight"] = (KV, E)
        out[f"{p}.self_attn.v_proj.weight"] = (KV, E)
        out[f"{p}.self_attn.o_proj.weight"] = (E, Q)
        out[f"{p}.post_attention_layernorm.weight"] = (E,)
        out[f"{p}.mlp.gate_proj.weight"] = (F, E)
        out[f"{p}.mlp.up_proj.weight"] = (F, E)
        out[f"{p}.mlp.down_proj.weight"] = (E, F)
    if not c.tie_word_embeddings:
        out["lm_head.weight"] = (V, E)
    return out


def random_device_weights(c: DecoderConfig, seed: int, device, std: float = 0.02) -> dict:
    """Random-init weights for ``c`` drawn on ``device``: matrices N(0, ``std``) in bf16, norm
    weights one (the ``--random-weights`` mode of iron/lm/cli.py:83-208 with the benchmark's
    deviation)."""
    import torch

    gen = torch.Generator(device=device).manual_seed(seed)
    out = {}
    for name, dims in checkpoint_shapes(c).items():
        if len(dims) >= 2:
            out[name] = (torch.randn(dims, generator=gen, device=device, dtype=torch.float32) * std).to(torch.bfloat16)
        else:
            out[name] = torch.ones(dims, device=device, dtype=torch.bfloat16)
    return out


def _llama():
    from ...lm.causal import CausalLM

    class Llama(CausalLM):
        """Llama 3 on ``config``'s shape and a checkpoint's ``weights``."""

        config_class = LlamaConfig
        profile = PROFILES

    return Llama


def __getattr__(name):
    # ``Llama`` needs the graph layer; keep the config importable without it
    if name == "Llama":
        cls = _llama()
        globals()["Llama"] = cls
        return cls
    raise AttributeError(name)


if __name__ == "__main__":
    import sys

    from ...lm.cli import main

    sys.exit(main(_llama()))
