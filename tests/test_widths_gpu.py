"""The fused engine at the real model widths against the oracle decoder (B200).

The toy shape of the golden tests never reaches the tile choices a real width takes: the
192/256-column CTA-pair tiles and the q/k/v projection with RoPE in its output stage
(hidden 2048 and 3072), the TMA-fed GEMV rings on 8192-wide rows, the key split of the
decode attention at a 2048-position hint, the 128-wide head of the 3B shape and a 128256-row
head.  Two layers of each width are enough to pass through every one of them: a ragged prompt
chunk of 320 tokens, then four teacher-forced decode steps, logits within 2 % of the largest
logit of the oracle's and the same greedy token wherever the oracle's own top two are
further apart than that bound.  The batched step (skinny split-K GEMMs, packed attention)
is held to the same oracle per sequence.
"""

import numpy as np
import pytest

from oracle import model as M
from tests.util import fast_random_weights

pytestmark = pytest.mark.gpu

WIDTHS = {
    "1B": dict(hidden_size=2048, num_attention_heads=32, num_key_value_heads=8, head_dim=64,
               intermediate_size=8192),
    "3B": dict(hidden_size=3072, num_attention_heads=24, num_key_value_heads=8, head_dim=128,
               intermediate_size=8192),
}


def shapes(width: str, max_seq_len: int, chunk: int):
    from iron_b200.applications.llama.model import Llama3RopeScaling, LlamaConfig

    common = dict(vocab_size=128256, num_hidden_layers=2, rope_theta=500000.0, max_seq_len=max_seq_len,
                  eps=1e-5, prefill_chunk=chunk, **WIDTHS[width])
    oracle = M.LlamaShape(rope_scaling=M.Llama3RopeScaling(32.0, 1.0, 4.0, 8192), **common)
    config = LlamaConfig(rope_scaling=Llama3RopeScaling(32.0, 1.0, 4.0, 8192), **common)
    return oracle, config


def close(got, want, what):
    """Within 2 % of the largest logit; the same token unless the oracle's top two are a near-tie."""
    got, want = np.asarray(got, np.float32), np.asarray(want, np.float32)
    bound = 0.02 * np.abs(want).max()
    err = np.abs(got - want).max()
    assert err <= bound, f"{what}: max error {err:.4g} over {bound:.4g}"
    top = np.sort(want)[-2:]
    if top[1] - top[0] > bound:
        assert int(got.argmax()) == int(want.argmax()), f"{what}: greedy token differs"
    else:
        assert want[int(got.argmax())] >= top[1] - bound, f"{what}: the drawn token is not a near-tie of the best"


@pytest.mark.parametrize("width", ["1B", "3B"])
def test_prompt_chunk_and_decode_steps_at_the_real_width(width):
    from iron_b200.lm.engine import LlamaEngine

    shape, config = shapes(width, 2304, 2048)
    weights = fast_random_weights(M.llama_shapes(shape), 11)
    engine = LlamaEngine(config, weights, kv_len_hint=2176)
    oracle = M.NumpyLlama(shape, weights)
    prompt = np.random.default_rng(21).integers(0, shape.vocab_size, 320)
    want = oracle.forward(prompt, 0)
    got = engine.prefill(prompt)
    close(got, want, f"{width} prompt chunk")
    tokens = list(prompt)
    for step in range(4):
        nxt = int(np.asarray(want, np.float32).argmax())
        want = oracle.forward([nxt], len(tokens))
        got = engine.feed([nxt], len(tokens))
        tokens.append(nxt)
        close(got, want, f"{width} decode step {step}")
    engine.check()


def test_batched_step_at_the_1b_width():
    from iron_b200.lm.engine import LlamaEngine

    shape, config = shapes("1B", 512, 256)
    weights = fast_random_weights(M.llama_shapes(shape), 12)
    nseq = 3
    engine = LlamaEngine(config, weights, batch=nseq, kv_len_hint=256)
    lengths = [130, 77, 201]
    firsts, wants = [], []
    for b, n in enumerate(lengths):
        prompt = np.random.default_rng(30 + b).integers(0, shape.vocab_size, n)
        oracle = M.NumpyLlama(shape, weights)
        first = oracle.forward(prompt, 0)
        close(engine.prefill(prompt, 0, seq=b), first, f"sequence {b} prompt")
        tok = int(np.asarray(first, np.float32).argmax())
        firsts.append(tok)
        wants.append(oracle.forward([tok], n))
    engine.set_batch(firsts, lengths)
    engine.step()
    got = engine.logits_batch()
    for b in range(nseq):
        close(got[b], wants[b], f"sequence {b} batched step")
    engine.check()
