"""Graphs without a device: per-call expressions, handle views, recording, host reference.

The contracts iron/tests/common/test_graph.py pins in the reference: what a per-call value
may and may not do (:534-600, :898-945), the Llama decode and prompt recordings
(:405-511: 18 steps a layer; 7 projection GEMMs a layer for a prompt chunk), errors
raised before any dispatch, and the model's host path against the reference's golden
logits (iron/tests/support/llama_reference.py:179-224).
"""

import dataclasses
from pathlib import Path

import numpy as np
import pytest
from ml_dtypes import bfloat16

import iron_b200 as iron
from iron_b200 import functional as F
from iron_b200.graph import Expr
from iron_b200.graph.expr import evaluate
from oracle import model as M
from tests.test_oracle_golden import assert_close

GOLDEN = Path(__file__).parent / "golden" / "llama_small.npz"


def test_per_call_expressions_are_closed_under_what_indices_need():
    p = Expr("position")
    assert (p + 1).evaluate({"position": 5}) == 6
    assert (p * 4 + 3).evaluate({"position": 5}) == 23
    assert ((p - 1) // 256 + 1).evaluate({"position": 600}) == 3
    assert (p // 4 // 8).evaluate({"position": 1000}) == 1000 // 32
    assert (p % 64).evaluate({"position": 130}) == 2
    assert (p + p * 2).evaluate({"position": 7}) == 21
    assert iron.clamp(p - 10, lo=0).evaluate({"position": 3}) == 0
    assert (p + 1).difference(p) == 1 and (p * 2).difference(p) is None
    for bad in (lambda: p // 3, lambda: p % 48, lambda: p < 3, lambda: bool(p), lambda: p * Expr("rows"),
                lambda: p + Expr("rows"), lambda: int(p), lambda: iron.clamp(p, hi=4) + 1):
        with pytest.raises(TypeError):
            bad()
    with pytest.raises(TypeError):
        (p + 1).evaluate({})


class FeedForward(iron.Graph):
    def __init__(self, E, H):
        self.norm = iron.param(E)
        self.gate, self.up, self.down = iron.param(H, E), iron.param(H, E), iron.param(E, H)
        self.cache = iron.state((16, E))

    def body(self, x, *, position: iron.Scratchpad[np.int32], rows: iron.Scratchpad[np.int32] = np.int32(1)):
        h = F.rms_norm(x, (x.shape[-1],), self.norm, 1e-5)
        y = x + F.linear(F.silu(F.linear(h, self.gate)) * F.linear(h, self.up), self.down)
        self.cache[position] = y.reshape(y.shape[-1])
        return y, iron.carry(position=position + 1)


def loaded(seed=0):
    rng = np.random.default_rng(seed)
    g = FeedForward(64, 128)
    g.load_state_dict({"norm": (1 + rng.standard_normal(64) / 10).astype(bfloat16),
                       "gate": (rng.standard_normal((128, 64)) / 8).astype(bfloat16),
                       "up": (rng.standard_normal((128, 64)) / 8).astype(bfloat16),
                       "down": (rng.standard_normal((64, 128)) / 11).astype(bfloat16)})
    return g, rng.standard_normal((1, 64)).astype(bfloat16)


def test_a_body_records_operator_steps_and_its_reference_runs_them():
    from oracle import ops

    g, x = loaded()
    rec = g.record(x=((1, 64), bfloat16))
    assert [s.op.name for s in rec.steps] == ["RMSNorm", "GEMV", "SiLU", "GEMV", "ElementwiseMul", "GEMV",
                                               "ElementwiseAdd", "Copy"]
    y, carried = g.reference(x, position=3)
    h = ops.rms_norm(x, np.asarray(g.norm), 1e-5)
    act = ops.mul(ops.silu(ops.gemv(np.asarray(g.gate), h[0])), ops.gemv(np.asarray(g.up), h[0]))
    want = ops.add(x, ops.gemv(np.asarray(g.down), act).reshape(1, 64))
    assert np.array_equal(y, want) and carried == {"position": 4}
    assert np.array_equal(g.cache.host.reshape(16, 64)[3], want[0])
    assert not g.cache.host.reshape(16, 64)[[0, 1, 2, 4]].astype(np.float32).any()


class EncoderMLP(iron.Graph):
    """The feed-forward half of an encoder layer: LayerNorm with bias, linear, GELU, linear, residual."""

    def __init__(self, E, H, approximate="none"):
        self.gamma, self.beta = iron.param(E), iron.param(E)
        self.fc1, self.b1, self.fc2 = iron.param(H, E), iron.param(H), iron.param(E, H)
        self.approximate = approximate

    def body(self, x):
        h = F.layer_norm(x, (x.shape[-1],), self.gamma, self.beta, 1e-5)
        return x + F.linear(F.gelu(F.linear(h, self.fc1, self.b1), self.approximate), self.fc2)


def loaded_encoder(approximate="none", rows=4, seed=1):
    rng = np.random.default_rng(seed)
    g = EncoderMLP(64, 128, approximate)
    g.load_state_dict({"gamma": (1 + rng.standard_normal(64) / 10).astype(bfloat16),
                       "beta": (rng.standard_normal(64) / 10).astype(bfloat16),
                       "fc1": (rng.standard_normal((128, 64)) / 8).astype(bfloat16),
                       "b1": (rng.standard_normal(128) / 10).astype(bfloat16),
                       "fc2": (rng.standard_normal((64, 128)) / 11).astype(bfloat16)})
    return g, rng.standard_normal((rows, 64)).astype(bfloat16)


@pytest.mark.parametrize("approximate", ["none", "tanh"])
def test_layer_norm_and_gelu_record_their_operators_and_follow_the_float64_formula(approximate):
    import math

    g, x = loaded_encoder(approximate)
    rec = g.record(x=((4, 64), bfloat16))
    names = [s.op.name for s in rec.steps]
    assert names[0] == "LayerNorm" and "GELU" in names and names.count("ProjectionGEMM") == 2
    y = g.reference(x)
    y = y[0] if isinstance(y, tuple) else y
    f = lambda a: np.asarray(a).astype(np.float64)
    xf = f(x)
    d = xf - xf.mean(-1, keepdims=True)
    h = d / np.sqrt((d * d).mean(-1, keepdims=True) + 1e-5) * f(g.gamma) + f(g.beta)
    u = h @ f(g.fc1).T + f(g.b1)
    if approximate == "none":
        a = 0.5 * u * (1 + np.vectorize(math.erf)(u / math.sqrt(2)))
    else:
        a = 0.5 * u * (1 + np.tanh(math.sqrt(2 / math.pi) * (u + 0.044715 * u ** 3)))
    want = xf + a @ f(g.fc2).T
    assert np.abs(f(y) - want).max() <= 6e-2     # a chain of bf16 roundings on values of a few units
    with pytest.raises(ValueError, match="neither 'tanh' nor 'none'"):
        loaded_encoder("fast")[0].record(x=((4, 64), bfloat16))


class ShortConv(iron.Graph):
    """A Mamba2 block's short conv: a prompt chunk of up to 8 rows, or one decode row."""

    def __init__(self, C, K, decode):
        self.taps = iron.param(K, C)
        self.carry = iron.state((K - 1, C))
        self.decode = decode

    def body(self, x, *, rows: iron.Scratchpad[np.int32] = np.int32(1)):
        state = F.ConvState(read=self.carry, write=self.carry)
        return F.causal_conv1d(x if self.decode else x[:rows], self.taps, state)


def conv_pair(C=64, K=4, seed=5):
    rng = np.random.default_rng(seed)
    taps = (rng.standard_normal((K, C)) / 2).astype(bfloat16)
    chunk, step = ShortConv(C, K, False), ShortConv(C, K, True)
    for g in (chunk, step):
        g.load_state_dict({"taps": taps})
    return chunk, step, taps, rng


def test_causal_conv_carries_its_last_rows_from_a_prompt_chunk_into_decode_steps():
    from oracle import ops

    chunk, step, taps, rng = conv_pair()
    assert [s.op.name for s in chunk.record(x=((8, 64), bfloat16)).steps] == ["CausalConv1d"]
    x = rng.standard_normal((8, 64)).astype(bfloat16)
    y = chunk.reference(x, rows=5)
    y = y[0] if isinstance(y, tuple) else y
    want, hist = ops.causal_conv1d(x[:5], taps, np.zeros((3, 64), bfloat16))
    assert np.array_equal(np.asarray(y)[:5].view(np.uint16), want.view(np.uint16))
    assert np.array_equal(chunk.carry.host.reshape(3, 64).view(np.uint16), np.asarray(hist).view(np.uint16))
    # a second, shorter chunk than the carry keeps part of the old carry
    y = chunk.reference(x, rows=2)
    want, hist2 = ops.causal_conv1d(x[:2], taps, hist)
    assert np.array_equal(chunk.carry.host.reshape(3, 64).view(np.uint16), np.asarray(hist2).view(np.uint16))
    # the one-row form sums the newest tap first; in float32 both orders agree to a rounding
    step.carry.host = np.array(chunk.carry.host)
    row = rng.standard_normal((1, 64)).astype(bfloat16)
    y1 = step.reference(row)
    y1 = y1[0] if isinstance(y1, tuple) else y1
    fwd, hist3 = ops.causal_conv1d(row, taps, hist2)
    assert np.abs(np.asarray(y1).astype(np.float32) - fwd.astype(np.float32)).max() <= 2e-2
    assert np.array_equal(step.carry.host.reshape(3, 64).view(np.uint16), np.asarray(hist3).view(np.uint16))
    with pytest.raises(ValueError, match="neither bounded per call nor one row"):
        step.record(x=((2, 64), bfloat16))


def test_bad_calls_are_refused_before_anything_runs():
    g, x = loaded()
    with pytest.raises(IndexError):
        g.reference(x, position=16)          # a row past the state
    with pytest.raises(TypeError):
        g.reference(x, position=1.5)         # per-call values are integers
    with pytest.raises(TypeError):
        g.reference(x)                       # a value without a default is needed
    with pytest.raises(TypeError):
        g.reference(x, position=1, tokens=3)  # an unknown value
    with pytest.raises(TypeError):
        FeedForward(64, 128).reference(x, position=0)  # params never loaded
    with pytest.raises(KeyError):
        FeedForward(64, 128).load_state_dict({})
    with pytest.raises(TypeError):
        g(x)                                 # a graph is compiled, or called in a body


def test_handle_views_carry_bounds_through_reshapes_and_refuse_what_is_not_a_view():
    class Views(iron.Graph):
        def __init__(self):
            self.table = iron.weight(np.arange(64 * 8, dtype=np.float32).reshape(64, 8).astype(bfloat16))
            self.log = {}

        def body(self, x, *, rows: iron.Scratchpad[np.int32], start: iron.Scratchpad[np.int32]):
            b = x[:rows]
            self.log["bound"] = b.valid
            self.log["merged"] = b.reshape(x.shape[0] * 2, x.shape[1] // 2).valid
            self.log["split"] = b.reshape(x.shape[0] * 2, x.shape[1] // 2).reshape(x.shape).valid
            run = self.table[start : start + 4]
            self.log["run"] = (run.shape, run.offset)
            for bad in (lambda: x[:, :4], lambda: x[::2], lambda: self.table[start : start * 2],
                        lambda: x[:rows][:rows]):
                with pytest.raises(TypeError):
                    bad()
            with pytest.raises(IndexError):
                x[99]
            return x

    from iron_b200.operators.copy import Copy

    v = Views()
    v.record(x=((8, 16), bfloat16))
    rows = Expr("rows")
    assert v.log["bound"] == {0: rows} and v.log["merged"] == {0: rows * 2} and v.log["split"] == {0: rows}
    assert v.log["run"][0] == (4, 8) and evaluate(v.log["run"][1], {"start": 5}) == 40


@pytest.fixture(scope="module")
def llama():
    from iron_b200.applications.llama.model import Llama, Llama3RopeScaling, LlamaConfig

    cfg = LlamaConfig(vocab_size=1024, hidden_size=512, num_hidden_layers=2, num_attention_heads=16,
                      num_key_value_heads=4, head_dim=64, intermediate_size=2048, rope_theta=500000.0,
                      max_seq_len=256, eps=1e-5, prefill_chunk=256,
                      rope_scaling=Llama3RopeScaling(8.0, 1.0, 4.0, 64))
    weights = M.filled_random(M.llama_shapes(M.SCALED), 0)
    with np.load(GOLDEN) as z:
        golden = {k: z[k] for k in z.files}
    return Llama, cfg, weights, golden


def test_llama_records_the_reference_step_sequence(llama):
    Llama, cfg, weights, _ = llama
    model = Llama(cfg, weights)
    decode = [s.op.name for s in model.record().steps]
    layer = ["RMSNorm", "GEMV", "GEMV", "GEMV", "RoPE", "RoPE", "Copy", "Copy", "MHA", "GEMV", "ElementwiseAdd",
             "RMSNorm", "GEMV", "SiLU", "GEMV", "ElementwiseMul", "GEMV", "ElementwiseAdd"]
    assert decode == ["Copy", "Copy"] + layer * 2 + ["RMSNorm", "GEMV", "Sample"]
    prompt = model.record(ids=((256,), np.int32)).steps
    assert sum(s.op.name == "ProjectionGEMM" for s in prompt) == 7 * 2      # seven a layer
    mha = next(s for s in prompt if s.op.name == "MHA")
    assert evaluate(mha.values["valid"], dict(rows=9, position=20)) == 9
    assert evaluate(mha.values["kv_valid"], dict(rows=9, position=20)) == 21


def test_llama_host_path_matches_the_oracle_bit_for_bit_and_the_golden_logits(llama):
    Llama, cfg, weights, golden = llama
    model = Llama(cfg, weights)
    oracle = M.NumpyLlama(M.SCALED, weights)
    prompt = np.random.default_rng(7).integers(0, 1024, 8)
    got = model.reference_logits(prompt)
    assert np.array_equal(got, oracle.forward(prompt, 0).astype(np.float32))
    assert_close(got, golden[M.golden_key(prompt)])
    tokens = prompt
    for step in range(3):
        nxt = int(golden[M.golden_key(tokens)].argmax())
        got = model.reference_logits([nxt], len(tokens))
        assert np.array_equal(got, oracle.forward([nxt], len(tokens)).astype(np.float32))
        tokens = np.append(tokens, nxt)
        assert_close(got, golden[M.golden_key(tokens)], f"step {step}")


def test_arena_plan_shares_transients_and_pins_residents():
    from iron_b200.arena import ArenaPlan, Live, place

    plan = ArenaPlan()
    sizes = {"w": 1000, "kv": 5000, "a": 4096, "b": 4096, "c": 4096}
    spans = plan.place_version([["a"], ["a", "b"], ["b", "c"], ["c"]], sizes, {"w": "W", "kv": "KV"})
    assert spans["a"].offset == spans["c"].offset                    # live ranges do not overlap
    assert not spans["a"].overlaps(spans["b"]) and not spans["b"].overlaps(spans["c"])
    fixed = [spans["w"], spans["kv"]]
    assert all(not t.overlaps(f) for t in (spans["a"], spans["b"], spans["c"]) for f in fixed)
    again = plan.place_version([["x"]], {"kv": 5000, "x": 64}, {"kv": "KV"})
    assert again["kv"].offset == spans["kv"].offset                  # one offset in every version
    with pytest.raises(ValueError):
        plan.place_version([[]], {"kv": 6000}, {"kv": "KV"})
    assert all(s.offset % 256 == 0 for s in (*spans.values(), *again.values()))
    # randomized: nothing live together ever overlaps
    rng = np.random.default_rng(0)
    for _ in range(20):
        n = int(rng.integers(2, 12))
        ranges = {f"t{i}": Live(*sorted(rng.integers(0, 10, 2).tolist())) for i in range(n)}
        szs = {k: int(rng.integers(1, 5000)) for k in ranges}
        placed, top = place(ranges, szs)
        for a in placed:
            for b in placed:
                if a < b and ranges[a].overlaps(ranges[b]):
                    assert not placed[a].overlaps(placed[b])
        assert top == max(s.end for s in placed.values())
