"""The one-kernel decode step against the separate launches and the oracle decoder (B200)."""

import numpy as np
import pytest

from oracle import model as M
from tests.test_engine_gpu import close_to_oracle, toy_config

pytestmark = pytest.mark.gpu


def engines(monkeypatch, config, weights, **kw):
    from iron_b200.lm.engine import LlamaEngine

    monkeypatch.setenv("IRON_DECODE_STEP", "1")
    fused = LlamaEngine(config, weights, **kw)
    monkeypatch.setenv("IRON_DECODE_STEP", "0")
    separate = LlamaEngine(config, weights, **kw)
    assert fused.fused_step and not separate.fused_step
    assert fused.launches_per_step == 1
    return fused, separate


def test_a_long_context_agrees_with_the_separate_launches(monkeypatch):
    """200 teacher-forced positions: every key batch and key split of the attention phase
    fills, and the two paths see the same caches."""
    weights = M.filled_random(M.llama_shapes(M.SCALED), 0)
    fused, separate = engines(monkeypatch, toy_config(), weights, kv_len_hint=200)
    tokens = np.random.default_rng(3).integers(0, 1024, 200)
    for at in (1, 7, 64, 65, 130, 200):
        lo = 0 if at == 1 else {7: 1, 64: 7, 65: 64, 130: 65, 200: 130}[at]
        a = fused.feed(tokens[lo:at], lo)
        b = separate.feed(tokens[lo:at], lo)
        # the key splits fold in a different order: a few bf16 ulps on the logits (each path is held to 2 % of the largest logit against the oracle)
        bound = float(np.abs(a - b).max())
        assert bound <= 0.02 * np.abs(b).max(), f"after {at} tokens"
        # the same greedy token wherever the leader is further ahead than the two paths differ
        top = np.sort(b)[-2:]
        if top[1] - top[0] > 2 * bound:
            assert int(a.argmax()) == int(b.argmax()), f"after {at} tokens"
    for l_f, l_s in zip(fused.layers, separate.layers):
        k_f, k_s = l_f["k"][0, :200].float(), l_s["k"][0, :200].float()
        assert (k_f - k_s).abs().max().item() <= 0.02 * k_s.abs().max().item()
    fused.check()


def test_the_device_carried_loop_draws_the_same_tokens(monkeypatch):
    weights = M.filled_random(M.llama_shapes(M.SCALED), 0)
    fused, separate = engines(monkeypatch, toy_config(), weights, kv_len_hint=64)
    prompt = np.random.default_rng(11).integers(0, 1024, 20)
    fused.feed(prompt[:-1], 0)
    separate.feed(prompt[:-1], 0)
    a = fused.generate(int(prompt[-1]), 19, 24)
    b = separate.generate(int(prompt[-1]), 19, 24)
    assert a == b
    assert int(fused.values[1].item()) == 19 + 24
    # and the step after a prompt run through the tensor-core path
    assert fused.complete(prompt, 8) == separate.complete(prompt, 8)


def test_head_dim_128_and_an_odd_head_count(monkeypatch):
    """The Llama-3.2-3B proportions scaled down: 128-wide heads, 6 heads over 2 KV heads
    (the key split does not divide the grid evenly), untied head."""
    from iron_b200.applications.llama.model import LlamaConfig

    shape = dict(vocab_size=2000, hidden_size=768, num_hidden_layers=2, num_attention_heads=6,
                 num_key_value_heads=2, head_dim=128, intermediate_size=1536, rope_theta=10000.0,
                 max_seq_len=128, eps=1e-5, prefill_chunk=128, tie_word_embeddings=False)
    config = LlamaConfig(**shape)
    spec = M.LlamaShape(**shape)
    weights = M.filled_random(M.llama_shapes(spec) | {"lm_head.weight": (2000, 768)}, 5)
    fused, separate = engines(monkeypatch, config, weights, kv_len_hint=100)
    tokens = np.random.default_rng(5).integers(0, 2000, 100)
    a, b = fused.feed(tokens, 0), separate.feed(tokens, 0)
    assert np.abs(a - b).max() <= 0.02 * np.abs(b).max()
    want = M.NumpyLlama(spec, weights).forward(tokens, 0).astype(np.float32)
    close_to_oracle(a, want, "100 tokens")
    fused.check()
