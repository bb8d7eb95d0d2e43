"""The fused decode engine against the oracle decoder and the reference's golden logits (B200)."""

import dataclasses
from pathlib import Path

import numpy as np
import pytest

from oracle import model as M
from tests.test_oracle_golden import assert_close

pytestmark = pytest.mark.gpu
GOLDEN = Path(__file__).parent / "golden" / "llama_small.npz"


def toy_config():
    from iron_b200.applications.llama.model import Llama3RopeScaling, LlamaConfig

    return LlamaConfig(
        vocab_size=1024, hidden_size=512, num_hidden_layers=2, num_attention_heads=16,
        num_key_value_heads=4, head_dim=64, intermediate_size=2048, rope_theta=500000.0,
        max_seq_len=256, eps=1e-5, prefill_chunk=256,
        rope_scaling=Llama3RopeScaling(8.0, 1.0, 4.0, 64))


@pytest.fixture(scope="module")
def case():
    from iron_b200.lm.engine import LlamaEngine

    weights = M.filled_random(M.llama_shapes(M.SCALED), 0)
    with np.load(GOLDEN) as z:
        golden = {k: z[k] for k in z.files}
    return LlamaEngine(toy_config(), weights, kv_len_hint=64), weights, golden


def test_decode_token_by_token_matches_the_golden_logits_and_the_oracle(case):
    engine, weights, golden = case
    prompt = np.random.default_rng(7).integers(0, 1024, 8)
    oracle = M.NumpyLlama(M.SCALED, weights)
    for i, t in enumerate(prompt):
        want = oracle.forward([t], i).astype(np.float32)
        got = engine.feed([t], i)
        # against the bf16 oracle: the north-star bound on bf16 logits
        err = np.abs(got - want)
        assert ((err <= 1e-2 * np.abs(want)) | (err <= 2e-2)).all(), f"position {i}: {err.max()}"
    assert_close(got, golden[M.golden_key(prompt)])
    # six greedy steps: logits close to the float32 judge's, same tokens
    tokens = prompt
    for step in range(6):
        nxt = int(golden[M.golden_key(tokens)].argmax())
        got = engine.feed([nxt], len(tokens))
        tokens = np.append(tokens, nxt)
        assert_close(got, golden[M.golden_key(tokens)], f"step {step}")


def test_device_carried_generation_draws_the_golden_tokens(case):
    engine, weights, golden = case
    prompt = np.random.default_rng(7).integers(0, 1024, 8)
    engine.feed(prompt[:-1], 0)
    drawn = engine.generate(int(prompt[-1]), len(prompt) - 1, 6)
    tokens, want = prompt, []
    for _ in range(6):
        want.append(int(golden[M.golden_key(tokens)].argmax()))
        tokens = np.append(tokens, want[-1])
    assert drawn == want
    # the host-driven step agrees with the device-carried loop, bit for bit
    engine.feed(prompt[:-1], 0)
    tok, host = int(prompt[-1]), []
    for i in range(6):
        tok = engine.decode(tok, len(prompt) - 1 + i)
        host.append(tok)
    assert host == want


def test_out_of_range_calls_are_refused_before_any_launch(case):
    engine, _, _ = case
    with pytest.raises(IndexError):
        engine.set_call(0, 256)
    with pytest.raises(IndexError):
        engine.set_call(1024, 0)
    with pytest.raises(IndexError):
        engine.generate(0, 250, 10)
