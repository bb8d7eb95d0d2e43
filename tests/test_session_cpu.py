"""Sessions over a causal model on the host (no GPU): history-aware logits, restarts, draws.

What iron/lm/session.py:32-126 does for the reference: one more token is a decode step, a
changed history restarts from the first token the caches do not hold -- or, with a Mamba2
mixer's recurrent state, from the prompt-chunk boundary before it
(tests/applications/granite_hybrid/reference/test.py:129-145) -- bad tokens and over-long
histories are refused before any dispatch, and sessions displace one another.
"""

import numpy as np
import pytest

from iron_b200.lm.causal import OnHost
from iron_b200.lm.generation import Sampler
from iron_b200.lm.session import Session
from oracle import model as M
from tests.models import toy
from tests.test_oracle_golden import assert_close


def host(name):
    cls, config, shape, weights, seed, golden = toy(name)
    model = type("Host" + cls.__name__, (OnHost, cls), {})(config, weights)
    return model, config, shape, weights, seed, golden


def test_one_more_token_is_a_decode_step_and_a_changed_history_restarts():
    model, config, shape, weights, seed, golden = host("granite")
    prompt = np.random.default_rng(seed).integers(0, 1024, 8)
    calls = []
    real = model.call_version
    model.call_version = lambda ids=None, **kw: (calls.append(("chunk" if ids is not None else "step", kw)), real(ids, **kw))[1]
    first = model.logits(prompt)
    assert_close(first, golden[M.golden_key(prompt)])
    assert [c[0] for c in calls] == ["chunk"] and calls[0][1]["rows"] == 8
    tokens = np.append(prompt, first.argmax())
    assert_close(model.logits(tokens), golden[M.golden_key(tokens)])
    assert calls[-1] == ("step", dict(token=int(tokens[-1]), position=8))
    # change token 5: positions 5.. are run again as one chunk from position 5
    changed = tokens.copy()
    changed[5] = (changed[5] + 1) % 1024
    model.logits(changed)
    assert calls[-1][0] == "chunk" and calls[-1][1]["start"] == 5 and calls[-1][1]["rows"] == 4
    assert np.array_equal(model.logits(changed), type(model)(config, weights).logits(changed))


def test_recurrent_states_restart_at_the_chunk_boundary_before_the_change():
    model, config, shape, weights, seed, golden = host("granite hybrid")
    assert len(model.recurrent) == 6      # a convolution state and a scan state per mixer
    tokens = np.random.default_rng(3).integers(0, config.vocab_size, 101)
    for position, start in ((0, 0), (64, 64), (70, 64), (100, 100)):
        model.logits(tokens[:100])
        model.forget(position)
        assert model.session._seen.size == start
        resumed = model.logits(tokens[: position + 1])
        fresh = type(model)(config, weights)     # the same calls from empty states
        if start:
            fresh.logits(tokens[:start])
        scratch = fresh.logits(tokens[: position + 1])
        # the same function of the same tokens; the host's float32 matrix products sum in an
        # order that depends on how many rows a call runs, so a flipped bf16 rounding is allowed
        assert np.abs(resumed - scratch).max() <= 0.01 * np.abs(scratch).max(), position
        assert resumed.argmax() == scratch.argmax()


def test_bad_histories_are_refused_and_leave_the_caches_as_they_were():
    model, config, *_ = host("granite")
    prompt = np.arange(8)
    before = model.logits(prompt)
    with pytest.raises(IndexError, match="outside"):
        model.logits([1, 2, 5000])
    with pytest.raises(ValueError, match="do not fit"):
        model.logits(np.zeros(config.max_seq_len + 1, np.int64))
    with pytest.raises(ValueError, match="do not fit"):
        model.logits([])
    assert model.session._seen.tolist() == prompt.tolist()
    assert np.array_equal(model.logits(np.append(prompt, 3)), type(model)(config, *host("granite")[3:4]).logits(np.append(prompt, 3)))
    del before


def test_sessions_displace_one_another():
    model, config, *_ = host("granite")
    a, b = model.session, Session(model)
    pa, pb = np.arange(1, 7), np.arange(20, 29)
    la = a.logits(pa)
    lb = b.logits(pb)
    assert model.holder is b
    assert np.array_equal(a.logits(pa), la) and model.holder is a      # run again from the first token
    assert np.array_equal(b.logits(pb), lb)


def test_generate_draws_the_golden_greedy_tokens_and_a_sampler_draws_as_the_host_would():
    model, config, shape, weights, seed, golden = host("granite")
    prompt = np.random.default_rng(seed).integers(0, 1024, 8)
    tokens, want = prompt, []
    for _ in range(5):
        want.append(int(golden[M.golden_key(tokens)].argmax()))
        tokens = np.append(tokens, want[-1])
    assert model.generate(prompt, 5) == want
    assert list(model.stream(prompt, 3)) == want[:3]
    # the session now holds the prompt and all drawn tokens but the last: one more is a step
    assert model.session._seen.tolist() == list(prompt) + want[:2]
    # sampled: the graph's Sample step reads the rows the sampler's uniforms filled, so it
    # draws what the host sampler draws from the same logits with the same uniforms
    drawn = model.generate(prompt, 4, Sampler(0.8, 20, seed=11))
    replay, history = Sampler(0.8, 20, seed=11), list(prompt)
    fresh = type(model)(config, weights)
    for t in drawn:
        assert replay(fresh.logits(history)) == t
        history.append(t)
    with pytest.raises(ValueError, match="do not fit"):
        model.generate(prompt, config.max_seq_len)
