"""Granite on the shared decoder (iron/applications/granite/model.py:32-96).

Granite is Llama's layer with four scalars from its config: the attention logits scaled by
``attention_multiplier``, each block's output by ``residual_multiplier`` before its
residual, the embedding rows by ``embedding_multiplier`` and the logits divided by
``logits_scaling``.  Its output head is its own matrix (``lm_head``).
"""

from __future__ import annotations

import dataclasses
import math

import numpy as np
from ml_dtypes import bfloat16

from ...graph import param
from ...lm.blocks import DecoderLayer
from ...lm.causal import CausalLM
from ...lm.config import DecoderConfig, Precision, not_json


@dataclasses.dataclass(frozen=True)
class GraniteConfig(DecoderConfig):
    """``DecoderConfig`` and Granite's four scalars."""

    attention_multiplier: float = dataclasses.field(kw_only=True)
    residual_multiplier: float = dataclasses.field(default=1.0, kw_only=True)
    embedding_multiplier: float = dataclasses.field(default=1.0, kw_only=True)
    logits_scaling: float = dataclasses.field(default=1.0, kw_only=True)
    precision: Precision = not_json(Precision.HIGH, kw_only=True)

    @property
    def attention_scale(self) -> float | None:
        return self.attention_multiplier


class GraniteLayer(DecoderLayer):
    """Llama's layer with the attention logits and each block's output scaled."""

    def __init__(self, c: GraniteConfig, i: int):
        super().__init__(c, i)
        self.self_attn.scaling = c.attention_multiplier
        self.residual_multiplier = c.residual_multiplier


class Granite(CausalLM):
    """Granite on ``config``'s shape and a checkpoint's ``weights``."""

    config_class = GraniteConfig
    layer_class = GraniteLayer

    def __init__(self, config: GraniteConfig, weights):
        super().__init__(config, weights)
        # the embedding's multiplier as a row every embedding row is multiplied by
        self.embed_scale = param(np.full(config.hidden_size, config.embedding_multiplier, bfloat16))
        if config.logits_scaling != 1:
            # the logits' divisor folded into the final norm's loaded weight, in bf16
            norm = self.model.norm
            norm.weight = param((np.asarray(norm.weight) / bfloat16(config.logits_scaling)).astype(bfloat16))

    def lookup(self, ids):
        x = super().lookup(ids)
        if self.config.embedding_multiplier == 1:
            return x
        E = self.config.hidden_size
        return x.reshape(math.prod(x.shape) // E, E) * self.embed_scale


if __name__ == "__main__":
    import sys

    from ...lm.cli import main

    sys.exit(main(Granite))
