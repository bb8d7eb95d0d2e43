"""The reference's other toy decoders compiled for the device (one CUDA graph per version)
against the reference's golden logits and the oracle decoder (B200).

Biased Llama (``Linear`` with a bias row), Granite (scaled attention logits, AXPY residuals,
the embedding-row product, the folded logits divisor) and the Granite 4.0-H hybrid, whose
three Mamba2 mixers run the causal-convolution and selective-scan kernels with their states
carried through ``Checkpoints`` slots from chunk to chunk and into decode steps.
"""

import dataclasses

import numpy as np
import pytest

from oracle import model as M
from tests.models import TOYS, toy
from tests.test_oracle_golden import assert_close

pytestmark = pytest.mark.gpu


def close_to_oracle(got, want, what):
    want = np.asarray(want, np.float32)
    err = np.abs(np.asarray(got, np.float32) - want).max()
    assert err <= 0.02 * np.abs(want).max(), f"{what}: max error {err:.4g}"
    assert int(np.argmax(got)) == int(np.argmax(want)), f"{what}: greedy token differs"


@pytest.fixture(scope="module", params=sorted(TOYS))
def case(request):
    return toy(request.param)


def test_prompt_then_greedy_steps_on_the_device(case):
    cls, config, shape, weights, seed, golden = case
    model, oracle = cls(config, weights), M.NumpyDecoder(shape, weights)
    prompt = np.random.default_rng(seed).integers(0, config.vocab_size, 8)
    got = model.logits(prompt)
    want = golden[M.golden_key(prompt)]
    assert_close(got, want)
    close_to_oracle(got, oracle.forward(prompt, 0), "prompt")
    tokens = prompt
    for step in range(6):
        tokens = np.append(tokens, want.argmax())
        got = model.logits(tokens[-1:], len(tokens) - 1)
        want = golden[M.golden_key(tokens)]
        assert_close(got, want, f"step {step}")
        close_to_oracle(got, oracle.forward(tokens[-1:], len(tokens) - 1), f"step {step}")


def test_a_prompt_of_several_chunks_then_a_step_then_a_turn_on_the_device(case):
    cls, config, _, weights, _, golden = case
    C = config.prefill_chunk
    model = cls(dataclasses.replace(config, max_seq_len=4 * C), weights)
    tokens = np.random.default_rng(3).integers(0, config.vocab_size, C + 150)
    first = golden[M.golden_key(tokens)]
    assert_close(model.logits(tokens), first)
    tokens = np.append(tokens, first.argmax())
    assert_close(model.logits(tokens[-1:], len(tokens) - 1), golden[M.golden_key(tokens)])
    turn = np.random.default_rng(4).integers(0, config.vocab_size, 30)
    restart = len(tokens) // C * C
    tokens = np.append(tokens, turn)
    assert_close(model.logits(tokens[restart:], restart), golden[M.golden_key(tokens)])
