"""The batched decode step (one row per sequence, each at its own position) against the
one-sequence engine and the oracle decoder (B200)."""

import numpy as np
import pytest

from oracle import model as M
from tests.test_engine_gpu import close_to_oracle, toy_config

pytestmark = pytest.mark.gpu


# the layer's RMSNorms, RoPE and cache write as launches of their own, or inside the projections
@pytest.fixture(scope="module", params=["0", "1", "norm", "rope"],
                ids=["separate kernels", "norm and rope folded in", "norm folded in", "rope folded in"])
def engines(request):
    from iron_b200.lm.engine import LlamaEngine

    weights = M.filled_random(M.llama_shapes(M.SCALED), 0)
    mp = pytest.MonkeyPatch()
    mp.setenv("IRON_DECODE_STEP", "0")
    mp.setenv("IRON_BATCH_FOLD", request.param)
    batched = LlamaEngine(toy_config(), weights, batch=3, kv_len_hint=64)
    single = LlamaEngine(toy_config(), weights, batch=1, kv_len_hint=64)
    mp.undo()
    assert batched.fold_norm == (request.param in ("1", "norm")) and batched.fold_rope == (request.param in ("1", "rope"))
    return batched, single, weights


def prompts():
    rng = np.random.default_rng(21)
    return [rng.integers(0, 1024, n) for n in (5, 12, 1)]


def test_rows_at_different_positions_match_the_one_sequence_engine_and_the_oracle(engines):
    batched, single, weights = engines
    ps = prompts()
    # every sequence but its last token goes through the prompt path of its own cache
    for b, p in enumerate(ps):
        if len(p) > 1:
            batched.prefill(p[:-1], 0, seq=b)
    tokens = [int(p[-1]) for p in ps]
    positions = [len(p) - 1 for p in ps]
    batched.set_batch(tokens, positions)
    batched.step()
    got = batched.logits_batch()
    for b, p in enumerate(ps):
        want_single = single.feed(p, 0)
        want_oracle = M.NumpyLlama(M.SCALED, weights).forward(p, 0).astype(np.float32)
        close_to_oracle(got[b], want_oracle, f"sequence {b} against the oracle")
        assert np.abs(got[b] - want_single).max() <= 0.02 * np.abs(want_single).max()
        assert int(got[b].argmax()) == int(want_single.argmax())
    # the step left (drawn token, position + 1) per sequence
    assert batched.b_pos.cpu().tolist() == [q + 1 for q in positions]
    assert batched.b_tokens.cpu().tolist() == [int(g.argmax()) for g in got]
    batched.check()


def test_the_device_carried_batched_loop_draws_each_sequences_tokens(engines):
    """Ten device-carried steps of three sequences at their own positions; every token drawn is
    the oracle decoder's greedy token for that sequence's history, or ties with it inside the
    logits' bound (two summation orders may break a near-tie differently; the history then
    follows the device's token)."""
    batched, _, weights = engines
    ps = prompts()
    for b, p in enumerate(ps):
        if len(p) > 1:
            batched.prefill(p[:-1], 0, seq=b)
    drawn = batched.generate_batch([int(p[-1]) for p in ps], [len(p) - 1 for p in ps], 10)
    assert drawn.shape == (3, 10)
    for b, p in enumerate(ps):
        oracle = M.NumpyLlama(M.SCALED, weights)
        logits = oracle.forward(p, 0).astype(np.float32)
        for step in range(10):
            tok = int(drawn[b, step])
            bound = 0.02 * np.abs(logits).max()
            assert logits[tok] >= logits.max() - bound, f"sequence {b} step {step}: token {tok} is not the oracle's"
            logits = oracle.forward([tok], len(p) + step).astype(np.float32)


def test_bad_batched_calls_are_refused_before_any_launch(engines):
    batched, _, _ = engines
    with pytest.raises(ValueError):
        batched.set_batch([1, 2], [0, 0])
    with pytest.raises(IndexError):
        batched.set_batch([1, 2, 3], [0, 0, 256])
    with pytest.raises(IndexError):
        batched.set_batch([1, 2, 1024], [0, 0, 0])
