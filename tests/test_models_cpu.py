"""The reference's other toy decoders recorded as this package's graphs and run on the host
(every recorded step's numpy ``reference()``), against the reference's golden float32 logits and
the oracle decoder (no GPU).

What iron/tests/support/llama_reference.py:179-224 checks of the reference's own host graphs:
decode token by token from empty states, a prompt then greedy steps, a prompt of several
chunks then a step and a turn.  The hybrid's Mamba2 mixers carry their convolution rows and
scan states across the chunk boundaries through ``Checkpoints``.
"""

import dataclasses

import numpy as np
import pytest

from oracle import model as M
from tests.models import TOYS, toy
from tests.test_oracle_golden import assert_close


@pytest.fixture(scope="module", params=sorted(TOYS))
def case(request):
    return toy(request.param)


def test_the_recorded_graph_on_the_host_matches_the_golden_rows_and_the_oracle_bit_for_bit(case):
    cls, config, shape, weights, seed, golden = case
    model, oracle = cls(config, weights), M.NumpyDecoder(shape, weights)
    prompt = np.random.default_rng(seed).integers(0, config.vocab_size, 8)
    got = model.reference_logits(prompt)
    want = golden[M.golden_key(prompt)]
    assert_close(got, want)
    assert np.array_equal(got, oracle.forward(prompt, 0).astype(np.float32))
    tokens = prompt
    for step in range(6):
        tokens = np.append(tokens, want.argmax())
        got = model.reference_logits(tokens[-1:], len(tokens) - 1)
        want = golden[M.golden_key(tokens)]
        assert_close(got, want, f"step {step}")
        assert np.array_equal(got, oracle.forward(tokens[-1:], len(tokens) - 1).astype(np.float32))


def test_decode_from_empty_states_token_by_token(case):
    cls, config, _, weights, seed, golden = case
    model = cls(config, weights)
    prompt = np.random.default_rng(seed).integers(0, config.vocab_size, 8)
    for i, t in enumerate(prompt):
        got = model.reference_logits([t], i)
    assert_close(got, golden[M.golden_key(prompt)])


def test_a_prompt_of_several_chunks_then_a_step_then_a_turn(case):
    cls, config, _, weights, _, golden = case
    C = config.prefill_chunk
    model = cls(dataclasses.replace(config, max_seq_len=4 * C), weights)
    tokens = np.random.default_rng(3).integers(0, config.vocab_size, C + 150)
    first = golden[M.golden_key(tokens)]
    assert_close(model.reference_logits(tokens), first)
    tokens = np.append(tokens, first.argmax())
    assert_close(model.reference_logits(tokens[-1:], len(tokens) - 1), golden[M.golden_key(tokens)])
    turn = np.random.default_rng(4).integers(0, config.vocab_size, 30)
    start = len(tokens)
    tokens = np.append(tokens, turn)
    # the turn reruns from the boundary of the chunk holding its first token, as the
    # reference's session does (iron/lm/session.py:32-59): chunks start on chunk boundaries
    restart = start // C * C
    assert_close(model.reference_logits(tokens[restart:], restart), golden[M.golden_key(tokens)])


def test_checkpoints_name_their_slots():
    from iron_b200.lm.causal import Checkpoints

    cp = Checkpoints.of((3, 8), 256, 64)
    assert cp.slots.shape == (5, 3, 8)
    assert [cp.slot(p) for p in (0, 1, 64, 65, 128, 256)] == [0, 1, 1, 2, 2, 4]
    assert cp.restart(100, 100) == 100 and cp.restart(100, 130) == 64 and cp.restart(64, 130) == 64
    with pytest.raises(ValueError, match="power of two"):
        Checkpoints.of((3, 8), 256, 48)


def test_the_hybrid_config_reads_its_checkpoint_and_refuses_experts():
    from iron_b200.applications.granite_hybrid.model import GraniteHybridConfig

    _, config, *_ = toy("granite hybrid")
    again = GraniteHybridConfig.from_json(config.to_json())   # prefill_chunk is no config.json field
    assert dataclasses.replace(again, prefill_chunk=64) == config and again.rope_theta is None and again.conv_channels == 16 * 64 + 2 * 2 * 64
    assert [again.attends(i) for i in range(4)] == [False, True, False, False]
    with pytest.raises(ValueError, match="dense sizes only"):
        dataclasses.replace(config, num_local_experts=8)
    with pytest.raises(ValueError, match="layer_types"):
        dataclasses.replace(config, num_hidden_layers=3)
