"""Pin the CPU oracle against the reference's own fixtures and formula tests (no GPU).

* the restated weight draw + config reproduce the reference's recorded float32 Hugging
  Face logits bit for bit (tests/golden/llama_small.npz, copied from
  iron/tests/common/goldens/small.npz by tests/golden/make_golden.py);
* the bf16 numpy decoder lies within the reference's own closeness bound of those rows
  (iron/lm/testing.py:190-206), token by token, whole prompt, and in chunks, as
  iron/tests/support/llama_reference.py:179-224 checks the reference's host graph;
* the RoPE convention and table formulas of
  iron/tests/operators/test_rope_reference_convention.py:22-59 and
  iron/tests/infrastructure/test_rope_angles.py hold for the restatements.
"""

import dataclasses
from pathlib import Path

import numpy as np
import pytest
from ml_dtypes import bfloat16

from oracle import model as M
from oracle import ops

GOLDEN = Path(__file__).parent / "golden" / "llama_small.npz"
LOGITS_SHARE = 0.05  # iron/lm/testing.py:187


def assert_close(got, want, what="the logits", share=LOGITS_SHARE):
    got = np.asarray(got, np.float32).reshape(want.shape)
    scale = np.abs(want).max()
    bound, err = share * scale, np.abs(got - want).max()
    assert err <= bound, f"{what}: max |diff| {err:.4f} against |logits| {scale:.3f}"
    second, first = np.sort(want, axis=None)[-2:]
    if first - second > bound:
        assert got.argmax() == want.argmax(), f"{what}: argmax differs"


@pytest.fixture(scope="module")
def golden():
    with np.load(GOLDEN) as z:
        return {k: z[k] for k in z.files}


@pytest.fixture(scope="module")
def toy():
    c = M.SCALED
    return c, M.filled_random(M.llama_shapes(c), 0)


def greedy_rows(golden, prompt, steps):
    tokens, rows = prompt, [golden[M.golden_key(prompt)]]
    for _ in range(steps):
        tokens = np.append(tokens, rows[-1].argmax())
        rows.append(golden[M.golden_key(tokens)])
    return tokens, rows


def test_float32_transformers_on_the_restated_draw_reproduces_the_golden_rows(golden, toy):
    c, w = toy
    hf = M.hf_llama(c, w)
    prompt = np.random.default_rng(7).integers(0, c.vocab_size, 8)
    tokens, rows = greedy_rows(golden, prompt, 2)
    for n, want in zip(range(len(prompt), len(tokens) + 1), rows):
        got = M.hf_logits(hf, tokens[:n])
        assert np.array_equal(got, want), f"{n} tokens: max diff {np.abs(got - want).max()}"


def test_numpy_decoder_prompt_then_decode_is_close_to_the_golden_rows(golden, toy):
    c, w = toy
    prompt = np.random.default_rng(7).integers(0, c.vocab_size, 8)
    tokens, rows = greedy_rows(golden, prompt, 6)
    model = M.NumpyLlama(c, w)
    got = model.forward(prompt, 0)
    assert_close(got, rows[0])
    for step in range(6):
        got = model.forward(tokens[len(prompt) + step : len(prompt) + step + 1], len(prompt) + step)
        assert_close(got, rows[step + 1], f"step {step}")


def test_numpy_decoder_token_by_token_from_an_empty_cache(golden, toy):
    c, w = toy
    prompt = np.random.default_rng(7).integers(0, c.vocab_size, 8)
    model = M.NumpyLlama(c, w)
    for i, t in enumerate(prompt):
        got = model.forward([t], i)
    assert_close(got, golden[M.golden_key(prompt)])


def test_numpy_decoder_runs_a_long_prompt_in_chunks(golden, toy):
    c, w = toy
    C = c.prefill_chunk
    c4 = dataclasses.replace(c, max_seq_len=4 * C)
    tokens = np.random.default_rng(3).integers(0, c.vocab_size, C + 150)
    want = golden[M.golden_key(tokens)]
    model = M.NumpyLlama(c4, w)
    assert_close(model.logits(tokens), want)
    tokens = np.append(tokens, want.argmax())
    assert_close(model.forward(tokens[-1:], len(tokens) - 1), golden[M.golden_key(tokens)])


def test_rope_is_block_major_with_interleaved_cos_sin():
    """iron/tests/operators/test_rope_reference_convention.py:22-59, row by row."""
    for rows, angle_rows in [(8, 2), (1024, 1), (4, 4), (13, 13), (12, 4)]:
        rng = np.random.default_rng(0)
        cols, half = 32, 16
        x = rng.standard_normal((rows, cols)).astype(bfloat16)
        angles = np.zeros((angle_rows, cols), dtype=bfloat16)
        angles[:, 0::2] = rng.random((angle_rows, half)).astype(bfloat16)
        angles[:, 1::2] = rng.random((angle_rows, half)).astype(bfloat16)
        want = np.empty((rows, cols), np.float32)
        for r in range(rows):
            a = r // (rows // angle_rows)
            cos, sin = angles[a, 0::2].astype(np.float32), angles[a, 1::2].astype(np.float32)
            x1, x2 = x[r, :half].astype(np.float32), x[r, half:].astype(np.float32)
            want[r, :half] = x1 * cos - x2 * sin
            want[r, half:] = x2 * cos + x1 * sin
        assert np.array_equal(want.astype(bfloat16), ops.rope(x, angles))


def test_rope_table_is_float64_trig_rounded_once():
    t = M.rope_angles(64, 128, 500000.0)
    inv = (1.0 / np.power(500000.0, (np.arange(0, 64, 2, dtype=np.float32) / np.float32(64)).astype(np.float64))).astype(np.float32)
    pos = 77
    want_cos = np.cos((np.float32(pos) * inv).astype(np.float32).astype(np.float64)).astype(np.float32)
    assert np.array_equal(t[pos, 0::2], want_cos)
    assert t.dtype == np.float32 and t.shape == (128, 64)
    assert np.all(t[0, 0::2] == 1) and np.all(t[0, 1::2] == 0)


def test_llama3_scaling_bands():
    """15 frequencies kept, 3 interpolated, 14 divided at the real 1B's scaling
    (iron/tests/infrastructure/test_rope_angles.py)."""
    s = M.Llama3RopeScaling(32.0, 1.0, 4.0, 8192)
    inv = 1.0 / np.power(500000.0, np.arange(0, 64, 2) / 64.0)
    out = s(inv)
    kept = np.isclose(out, inv, rtol=0, atol=0)
    divided = np.isclose(out, inv / 32.0, rtol=1e-15)
    assert kept.sum() == 15 and divided.sum() == 14 and (~kept & ~divided).sum() == 3


def test_leaf_formulas_match_plain_numpy():
    """RMSNorm as iron/tests/lm/test_modules.py:204-206 states it, within its 5 %."""
    rng = np.random.default_rng(0)
    x = rng.standard_normal((4, 256)).astype(bfloat16)
    w = (1 + rng.standard_normal(256) / 10).astype(bfloat16)
    xf, wf = x.astype(np.float32), w.astype(np.float32)
    want = xf / np.sqrt(np.mean(xf**2, -1, keepdims=True) + 1e-5) * wf
    got = ops.rms_norm(x, w, 1e-5).astype(np.float32)
    assert np.abs(got - want).max() <= 0.05 * np.abs(want).max()


def test_mha_rows_past_s_q_are_zero_and_keys_past_s_kv_masked():
    """iron/operators/mha.py:1076-1096 and iron/tests/operators/test_mha_bounded_rows.py:99-111."""
    rng = np.random.default_rng(1)
    H, G, S, D = 4, 2, 16, 64
    q = rng.standard_normal((S, H, D)).astype(bfloat16)
    k = rng.standard_normal((S, G, D)).astype(bfloat16)
    v = rng.standard_normal((S, G, D)).astype(bfloat16)
    full = ops.mha(q, k, v, num_heads=H, num_kv_heads=G, heads_interleaved=True, kv_interleaved=True)
    part = ops.mha(q, k, v, num_heads=H, num_kv_heads=G, heads_interleaved=True, kv_interleaved=True,
                   q_tokens=5, kv_tokens=5)
    assert np.array_equal(part[:5], full[:5])  # causal: the first rows see the same keys
    assert not part[5:].astype(np.float32).any()


def test_selective_scan_decays_and_reads_out():
    rng = np.random.default_rng(3)
    H, P, N = 2, 16, 16
    xbc = (rng.standard_normal((5, H * P + 2 * N)) * 0.5).astype(bfloat16)
    dt = rng.standard_normal((5, H)).astype(bfloat16)
    head = np.stack([rng.uniform(-4, 0, H), -rng.uniform(0.5, 16, H), rng.uniform(0, 2, H)], 1).astype(np.float32)
    state = rng.standard_normal((H, P, N)).astype(np.float32)
    y, final = ops.selective_scan(xbc, dt, head, state, heads=H, head_dim=P, state_size=N)
    y1, mid = ops.selective_scan(xbc[:3], dt[:3], head, state, heads=H, head_dim=P, state_size=N)
    y2, final2 = ops.selective_scan(xbc[3:], dt[3:], head, mid, heads=H, head_dim=P, state_size=N)
    assert np.array_equal(y, np.concatenate([y1, y2])) and np.allclose(final, final2)


# ---------------------------------------------------------------------------------------
# The reference's other toy decoders: biased Llama, Granite, and the Granite 4.0-H hybrid,
# whose golden is the one fixture that pins the selective scan and the causal convolution.

OTHER_TOYS = {
    # name: (shape, transformers model_type, prompt seed, fixture, float32 slack)
    "biased": (M.BIASED, "llama", 1, "llama_biased.npz", 0.0),
    "granite": (M.GRANITE_TOY, "granite", 0, "granite_toy.npz", 0.0),
    # transformers' Mamba2 mixer off its fused kernels sums in an order that depends on the
    # build: float32 rounding (2e-7 of logits up to 0.44) is all that separates the rows
    "hybrid": (M.HYBRID_TOY, "granitemoehybrid", 2, "granite_hybrid_dense.npz", 1e-6),
}


@pytest.fixture(scope="module", params=sorted(OTHER_TOYS))
def other(request):
    c, model_type, seed, fixture, slack = OTHER_TOYS[request.param]
    w = M.filled_random(M.decoder_shapes(c), 0)
    if c.layer_types is not None:
        w = M.hybrid_redraw(c, w)
    with np.load(Path(__file__).parent / "golden" / fixture) as z:
        rows = {k: z[k] for k in z.files}
    return c, w, model_type, seed, rows, slack


def test_float32_transformers_reproduces_the_other_toys_golden_rows(other):
    c, w, model_type, seed, golden, slack = other
    hf = M.hf_decoder(model_type, c, w)
    prompt = np.random.default_rng(seed).integers(0, c.vocab_size, 8)
    tokens, rows = greedy_rows(golden, prompt, 2)
    for n, want in zip(range(len(prompt), len(tokens) + 1), rows):
        got = M.hf_logits(hf, tokens[:n])
        assert np.abs(got - want).max() <= slack, f"{n} tokens: max diff {np.abs(got - want).max()}"
        assert got.argmax() == want.argmax()


def test_the_numpy_decoder_of_the_other_toys_is_close_to_their_golden_rows(other):
    """Prompt then six greedy steps, token by token from empty states, and a prompt of several
    chunks followed by a decode step and a turn of thirty tokens (the mixers' convolution
    history and scan state cross chunk boundaries): iron/tests/support/llama_reference.py:179-224."""
    c, w, _, seed, golden, _ = other
    prompt = np.random.default_rng(seed).integers(0, c.vocab_size, 8)
    tokens, rows = greedy_rows(golden, prompt, 6)
    model = M.NumpyDecoder(c, w)
    assert_close(model.forward(prompt, 0), rows[0])
    for step in range(6):
        at = len(prompt) + step
        assert_close(model.forward(tokens[at : at + 1], at), rows[step + 1], f"step {step}")
    model = M.NumpyDecoder(c, w)
    for i, t in enumerate(prompt):
        got = model.forward([t], i)
    assert_close(got, rows[0], "token by token")
    C = c.prefill_chunk
    long = np.random.default_rng(3).integers(0, c.vocab_size, C + 150)
    want = golden[M.golden_key(long)]
    model = M.NumpyDecoder(dataclasses.replace(c, max_seq_len=4 * C), w)
    assert_close(model.logits(long), want, "several chunks")
    long = np.append(long, want.argmax())
    assert_close(model.forward(long[-1:], len(long) - 1), golden[M.golden_key(long)], "the step after")
    turn = np.random.default_rng(4).integers(0, c.vocab_size, 30)
    start = len(long)
    long = np.append(long, turn)
    assert_close(model.forward(turn, start), golden[M.golden_key(long)], "a turn of thirty tokens")
