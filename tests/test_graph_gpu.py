"""Compiled graphs on the device against their own host reference and the golden logits (B200)."""

from pathlib import Path

import numpy as np
import pytest
from ml_dtypes import bfloat16

from oracle import model as M
from tests.test_graph_cpu import FeedForward, conv_pair, loaded, loaded_encoder
from tests.test_oracle_golden import assert_close

pytestmark = pytest.mark.gpu
GOLDEN = Path(__file__).parent / "golden" / "llama_small.npz"


def test_a_compiled_graph_replays_with_new_per_call_values():
    g, x = loaded()
    ref, _ = loaded()
    version = g.compile(x=((1, 64), bfloat16))
    for position in (3, 7, 3, 15):
        y, carried = version(x, position=position)
        want, want_carried = ref.reference(x, position=position)
        got = y.numpy().astype(np.float32)
        assert np.abs(got - want.astype(np.float32)).max() <= 2e-2 and carried == want_carried
        x = (x.astype(np.float32) * 0.5 + 0.1).astype(bfloat16)
    cache = version.read(g.cache).astype(np.float32)
    want_cache = ref.cache.host.reshape(16, 64).astype(np.float32)
    assert np.abs(cache - want_cache).max() <= 2e-2
    assert not cache[[0, 1, 2, 4, 5, 6]].any()
    assert g.compile(x=((1, 64), bfloat16)) is version
    with pytest.raises(ValueError, match="a new shape is a new compile"):
        version(np.zeros((2, 64), bfloat16), position=0)
    with pytest.raises(TypeError):
        version(x.astype(np.float32), position=0)
    with pytest.raises(IndexError):
        version(x, position=16)
    with pytest.raises(TypeError):
        version(x)


@pytest.mark.parametrize("approximate", ["none", "tanh"])
def test_an_encoder_feed_forward_runs_layer_norm_and_gelu_on_the_device(approximate):
    g, x = loaded_encoder(approximate)
    ref, _ = loaded_encoder(approximate)
    version = g.compile(x=((4, 64), bfloat16))
    out = version(x)
    y = out[0] if isinstance(out, tuple) else out
    want = ref.reference(x)
    want = want[0] if isinstance(want, tuple) else want
    assert np.abs(y.numpy().astype(np.float32) - np.asarray(want).astype(np.float32)).max() <= 3e-2


def test_causal_conv_graph_carries_rows_between_calls_bit_for_bit():
    chunk, step, taps, rng = conv_pair()
    ref_chunk, ref_step, _, _ = conv_pair()
    bits = lambda a: np.ascontiguousarray(np.asarray(a)).view(np.uint16)
    first = lambda out: out[0] if isinstance(out, tuple) else out
    cv = chunk.compile(x=((8, 64), bfloat16))
    x = rng.standard_normal((8, 64)).astype(bfloat16)
    for rows in (5, 2, 8):
        got = first(cv(x, rows=rows)).numpy()
        want = np.asarray(first(ref_chunk.reference(x, rows=rows)))
        assert np.array_equal(bits(got[:rows]), bits(want[:rows])) and not got[rows:].astype(np.float32).any()
        assert np.array_equal(bits(cv.read(chunk.carry)), bits(ref_chunk.carry.host.reshape(3, 64)))
        x = (x.astype(np.float32) * 0.5 - 0.25).astype(bfloat16)
    sv = step.compile(x=((1, 64), bfloat16))
    for _ in range(4):
        row = rng.standard_normal((1, 64)).astype(bfloat16)
        got = first(sv(row)).numpy()
        want = np.asarray(first(ref_step.reference(row)))
        assert np.array_equal(bits(got), bits(want))
        assert np.array_equal(bits(sv.read(step.carry)), bits(ref_step.carry.host.reshape(3, 64)))


def test_llama_compiled_graphs_match_the_golden_logits_prompt_then_decode():
    from iron_b200.applications.llama.model import Llama, Llama3RopeScaling, LlamaConfig

    cfg = LlamaConfig(vocab_size=1024, hidden_size=512, num_hidden_layers=2, num_attention_heads=16,
                      num_key_value_heads=4, head_dim=64, intermediate_size=2048, rope_theta=500000.0,
                      max_seq_len=256, eps=1e-5, prefill_chunk=256,
                      rope_scaling=Llama3RopeScaling(8.0, 1.0, 4.0, 64))
    weights = M.filled_random(M.llama_shapes(M.SCALED), 0)
    with np.load(GOLDEN) as z:
        golden = {k: z[k] for k in z.files}
    model = Llama(cfg, weights)
    prompt = np.random.default_rng(7).integers(0, 1024, 8)
    got = model.logits(prompt)
    assert_close(got, golden[M.golden_key(prompt)])
    host = Llama(cfg, weights).reference_logits(prompt)
    assert np.abs(got - host).max() <= 0.02 * np.abs(host).max() and got.argmax() == host.argmax()
    tokens = prompt
    for step in range(6):
        nxt = int(golden[M.golden_key(tokens)].argmax())
        got = model.logits([nxt], len(tokens))
        tokens = np.append(tokens, nxt)
        assert_close(got, golden[M.golden_key(tokens)], f"step {step}")
    # the two versions share one arena: the prompt's caches are the decode step's
    assert len(model.__dict__["_versions"]) == 2
    # the fused engine on the same weights draws the same greedy tokens
    engine = model.engine(kv_len_hint=64)
    want = []
    tokens = prompt
    for _ in range(4):
        want.append(int(golden[M.golden_key(tokens)].argmax()))
        tokens = np.append(tokens, want[-1])
    assert engine.complete(prompt, 4) == want


def test_check_mode_runs_every_step_alone_and_names_the_step_that_is_wrong(monkeypatch):
    """``compile(check=True)``: each step of the toy Llama's decode step and prompt chunk is
    launched on its own and held to its ``reference()`` on the inputs the device read; then one
    operator's launch is sabotaged and the check names that step."""
    from iron_b200.applications.llama.model import Llama, Llama3RopeScaling, LlamaConfig
    from iron_b200.graph import StepCheckFailed
    from iron_b200.operators.silu import SiLU

    cfg = LlamaConfig(vocab_size=1024, hidden_size=512, num_hidden_layers=2, num_attention_heads=16,
                      num_key_value_heads=4, head_dim=64, intermediate_size=2048, rope_theta=500000.0,
                      max_seq_len=256, eps=1e-5, prefill_chunk=256,
                      rope_scaling=Llama3RopeScaling(8.0, 1.0, 4.0, 64))
    weights = M.filled_random(M.llama_shapes(M.SCALED), 0)
    model = Llama(cfg, weights)
    ids = np.zeros(256, np.int32)
    ids[:8] = np.random.default_rng(7).integers(0, 1024, 8)
    chunk = model.compile(check=True, ids=((256,), np.int32))
    assert chunk is not model.compile(ids=((256,), np.int32))
    logits, carried = chunk(ids, position=7, start=0, rows=8)
    step = model.compile(check=True)
    logits2, carried2 = step(token=carried["token"], position=8)
    assert carried2["position"] == 9
    # break SiLU's launch: its output stays whatever the buffer held
    monkeypatch.setattr(SiLU, "launch", lambda self, buffers, values: None)
    with pytest.raises(StepCheckFailed, match="SiLU"):
        step(token=carried["token"], position=9)
