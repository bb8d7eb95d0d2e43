"""The fused decode engine against the oracle decoder and the reference's golden logits (B200)."""

import dataclasses
from pathlib import Path

import numpy as np
import pytest

from oracle import model as M
from tests.test_oracle_golden import assert_close

pytestmark = pytest.mark.gpu


def close_to_oracle(got, want, what=""):
    """bf16 logits against the bf16 oracle decoder.

    A logit is a 512-term dot product of activations that already passed through every
    layer, so a one-ulp rounding flip upstream moves it by an amount set by the logits'
    scale, not by its own size: the bound is 2 % of the largest logit (the reference holds
    its own graphs to 5 % of it against float32, iron/lm/testing.py:187), and the greedy
    token must agree.  Each operator alone is held to 1e-2 / 2e-2 in the kernel tests."""
    want = np.asarray(want, np.float32)
    err = np.abs(np.asarray(got, np.float32) - want)
    assert err.max() <= 0.02 * np.abs(want).max(), f"{what}: max error {err.max():.4g}"
    assert int(np.argmax(got)) == int(np.argmax(want)), f"{what}: greedy token differs"


GOLDEN = Path(__file__).parent / "golden" / "llama_small.npz"


def toy_config():
    from iron_b200.applications.llama.model import Llama3RopeScaling, LlamaConfig

    return LlamaConfig(
        vocab_size=1024, hidden_size=512, num_hidden_layers=2, num_attention_heads=16,
        num_key_value_heads=4, head_dim=64, intermediate_size=2048, rope_theta=500000.0,
        max_seq_len=256, eps=1e-5, prefill_chunk=256,
        rope_scaling=Llama3RopeScaling(8.0, 1.0, 4.0, 64))


@pytest.fixture(scope="module", params=["one-kernel step", "five launches a layer", "four launches a layer"])
def case(request):
    """The engine on each of its decode paths: the persistent one-kernel step, the separate
    launches per projection (what batches and tensor-parallel shards take), and the default,
    a layer's attention and o_proj as one launch."""
    from iron_b200.lm.engine import LlamaEngine

    mp = pytest.MonkeyPatch()
    mp.setenv("IRON_DECODE_STEP", "1" if request.param == "one-kernel step" else "0")
    mp.setenv("IRON_ATTN_OPROJ", "1" if request.param == "four launches a layer" else "0")
    request.addfinalizer(mp.undo)
    weights = M.filled_random(M.llama_shapes(M.SCALED), 0)
    with np.load(GOLDEN) as z:
        golden = {k: z[k] for k in z.files}
    engine = LlamaEngine(toy_config(), weights, kv_len_hint=64)
    assert engine.attn_oproj == (request.param == "four launches a layer")
    return engine, weights, golden


def test_decode_token_by_token_matches_the_golden_logits_and_the_oracle(case):
    engine, weights, golden = case
    prompt = np.random.default_rng(7).integers(0, 1024, 8)
    oracle = M.NumpyLlama(M.SCALED, weights)
    for i, t in enumerate(prompt):
        want = oracle.forward([t], i).astype(np.float32)
        got = engine.feed([t], i)
        close_to_oracle(got, want, f"position {i}")
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


def test_the_prompt_in_one_chunk_matches_the_golden_logits_and_leaves_decode_its_caches(case):
    engine, weights, golden = case
    prompt = np.random.default_rng(7).integers(0, 1024, 8)
    oracle = M.NumpyLlama(M.SCALED, weights)
    want = oracle.forward(prompt, 0).astype(np.float32)
    got = engine.prefill(prompt)
    close_to_oracle(got, want, "prompt")
    assert_close(got, golden[M.golden_key(prompt)])
    tokens = prompt
    for step in range(6):  # decode continues from the caches the prompt wrote
        nxt = int(golden[M.golden_key(tokens)].argmax())
        got = engine.feed([nxt], len(tokens))
        tokens = np.append(tokens, nxt)
        assert_close(got, golden[M.golden_key(tokens)], f"step {step}")


def test_complete_draws_the_golden_tokens_from_a_prompt(case):
    engine, weights, golden = case
    prompt = np.random.default_rng(7).integers(0, 1024, 8)
    tokens, want = prompt, []
    for _ in range(7):
        want.append(int(golden[M.golden_key(tokens)].argmax()))
        tokens = np.append(tokens, want[-1])
    assert engine.complete(prompt, 7) == want


def test_a_prompt_longer_than_a_chunk_runs_in_chunks(case):
    from iron_b200.lm.engine import LlamaEngine

    _, weights, golden = case
    config = dataclasses.replace(toy_config(), max_seq_len=1024, prefill_chunk=256)
    engine = LlamaEngine(config, weights, kv_len_hint=512)
    tokens = np.random.default_rng(3).integers(0, 1024, 256 + 150)
    first = golden[M.golden_key(tokens)]
    assert_close(engine.prefill(tokens), first)
    tokens = np.append(tokens, first.argmax())
    assert_close(engine.feed(tokens[-1:], len(tokens) - 1), golden[M.golden_key(tokens)])
    turn = np.random.default_rng(4).integers(0, 1024, 30)
    start = len(tokens)
    tokens = np.append(tokens, turn)
    assert_close(engine.prefill(turn, start), golden[M.golden_key(tokens)])


def test_prompt_rows_outside_the_caches_are_refused(case):
    engine, _, _ = case
    with pytest.raises(IndexError):
        engine.prefill_chunk([1, 2, 3], 255)
    with pytest.raises(IndexError):
        engine.prefill_chunk([1, 5000], 0)
    with pytest.raises(ValueError):
        engine.prefill_chunk([], 0)


def test_a_sliding_window_config_matches_the_host_graph_in_prompt_and_decode():
    """``sliding_window`` in the config bounds every layer's attention (iron/lm/blocks.py:504-529):
    the engine's prompt chunk (160 tokens: the tcgen05 attention with a window) and its decode
    steps against the host path, every recorded operator's numpy reference."""
    import dataclasses as dc

    from iron_b200.applications.llama.model import Llama
    from iron_b200.lm.engine import LlamaEngine

    config = dc.replace(toy_config(), sliding_window=48)
    assert config.window == 47
    weights = M.filled_random(M.llama_shapes(M.SCALED), 0)
    prompt = np.random.default_rng(12).integers(0, 1024, 160)
    engine = LlamaEngine(config, weights, kv_len_hint=200)
    host = Llama(config, weights)
    got = engine.prefill(prompt)
    want = host.reference_logits(prompt, 0)
    close_to_oracle(got, want, "windowed prompt")
    # the window matters: the same prompt without it gives other logits
    full = LlamaEngine(toy_config(), weights, kv_len_hint=200).prefill(prompt)
    assert np.abs(full - got).max() > 0.05 * np.abs(got).max()
    tokens = list(prompt)
    for step in range(3):
        nxt = int(np.argmax(want))
        got = engine.feed([nxt], len(tokens))
        want = host.reference_logits([nxt], len(tokens))
        tokens.append(nxt)
        close_to_oracle(got, want, f"windowed decode step {step}")


def test_stepping_stops_at_the_end_of_the_caches():
    """The carried loop is refused on the host at the last cache row, and the kernels hold a
    device-carried position inside the caches even when replayed without the host's check."""
    import torch

    from iron_b200.lm.engine import LlamaEngine

    config = dataclasses.replace(toy_config(), max_seq_len=16, prefill_chunk=16)
    weights = M.filled_random(M.llama_shapes(M.SCALED), 0)
    engine = LlamaEngine(config, weights, kv_len_hint=16)
    engine.set_call(3, 13)
    engine.step(); engine.step(); engine.step()          # positions 13, 14, 15: the last row
    with pytest.raises(IndexError):
        engine.step()
    with pytest.raises(IndexError):
        engine.generate(3, 14, 3)
    torch.cuda.synchronize()
    assert int(engine.values[1].item()) == 16
    # a raw replay past the end (what a caller holding the graph could do): nothing outside
    # the caches and the drawn row changes, and the position stays at the end
    before = engine.arena.clone()
    engine._graph.replay()
    torch.cuda.synchronize()
    assert int(engine.values[1].item()) == 16
    changed = (engine.arena != before).nonzero().flatten()
    drawn_lo = engine.drawn.data_ptr() - engine.arena.data_ptr()
    assert not ((changed >= drawn_lo) & (changed < drawn_lo + engine.drawn.numel() * 4)).any()
    for l in engine.layers:   # only the last cache row may have been rewritten
        for c in (l["k"], l["v"]):
            lo = c.data_ptr() - engine.arena.data_ptr()
            inside = changed[(changed >= lo) & (changed < lo + c.numel() * 2)]
            assert ((inside - lo) // (c.shape[2] * c.shape[3] * 2) == 15).all()
