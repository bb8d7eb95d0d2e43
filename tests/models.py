"""The reference's toy decoders as this package's graphs, with their drawn weights and goldens."""

from pathlib import Path

import numpy as np

from oracle import model as M

GOLDENS = Path(__file__).parent / "golden"


def biased_llama():
    from iron_b200.applications.llama.model import Llama, LlamaConfig

    c = M.BIASED
    config = LlamaConfig(vocab_size=c.vocab_size, hidden_size=c.hidden_size, num_hidden_layers=c.num_hidden_layers,
                         num_attention_heads=c.num_attention_heads, num_key_value_heads=c.num_key_value_heads,
                         head_dim=c.head_dim, intermediate_size=c.intermediate_size, rope_theta=c.rope_theta,
                         max_seq_len=c.max_seq_len, eps=c.eps, prefill_chunk=c.prefill_chunk, attention_bias=True)
    return Llama, config, c, 1, "llama_biased.npz"


def granite():
    from iron_b200.applications.granite.model import Granite, GraniteConfig

    c = M.GRANITE_TOY
    config = GraniteConfig(vocab_size=1024, hidden_size=512, num_hidden_layers=2, num_attention_heads=8,
                           num_key_value_heads=2, intermediate_size=1024, rope_theta=10000.0, max_seq_len=256,
                           prefill_chunk=256, tie_word_embeddings=False, attention_multiplier=0.0625,
                           residual_multiplier=0.22, embedding_multiplier=12.0, logits_scaling=8.0)
    return Granite, config, c, 0, "granite_toy.npz"


def granite_hybrid():
    from iron_b200.applications.granite_hybrid.model import GraniteHybrid, GraniteHybridConfig

    c = M.HYBRID_TOY
    config = GraniteHybridConfig(
        vocab_size=1024, hidden_size=512, num_hidden_layers=4, num_attention_heads=8, num_key_value_heads=2,
        intermediate_size=256, max_seq_len=256, prefill_chunk=64, attention_multiplier=0.0625,
        residual_multiplier=0.22, embedding_multiplier=12.0, logits_scaling=8.0, tie_word_embeddings=False,
        layer_types=("mamba", "attention", "mamba", "mamba"), position_embedding_type="nope",
        shared_intermediate_size=512, num_local_experts=0, num_experts_per_tok=2, mamba_n_heads=16,
        mamba_d_head=64, mamba_d_state=64, mamba_n_groups=2)
    return GraniteHybrid, config, c, 2, "granite_hybrid_dense.npz"


TOYS = {"biased llama": biased_llama, "granite": granite, "granite hybrid": granite_hybrid}


def toy(name: str):
    """(model class, its config, the oracle's shape, drawn weights, prompt seed, golden rows)."""
    cls, config, shape, seed, fixture = TOYS[name]()
    weights = M.filled_random(M.decoder_shapes(shape), 0)
    if shape.layer_types is not None:
        weights = M.hybrid_redraw(shape, weights)
    with np.load(GOLDENS / fixture) as z:
        golden = {k: z[k] for k in z.files}
    return cls, config, shape, weights, seed, golden
