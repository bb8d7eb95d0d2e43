"""The host sampler without a device: the rule of iron_b200/lm/generation.py.

The class contract follows iron/lm/generation.py:24-94 (temperature, then top-k, then a draw;
``rows`` takes the uniforms the host draws would; greedy at temperature 0).  The arithmetic
is this package's own rule, since the reference's lives outside its tree: these tests hold
the rule's pieces to exact values and to the float64 softmax.
"""

import numpy as np
import pytest
from ml_dtypes import bfloat16

from iron_b200.lm.generation import (K_MAX, ROW_WORDS, Sampler, candidates, draw_row, exp2_det, greedy,
                                     ordered_keys, sample_ref, sample_weights)


def test_candidates_order_by_value_then_index_with_nan_last():
    x = np.array([1.0, 3.0, -0.0, 3.0, np.nan, 0.0, -2.0, 3.0], np.float32).astype(bfloat16)
    assert candidates(x, 8).tolist() == [1, 3, 7, 0, 5, 2, 6, 4]      # +0 above -0, NaN last
    assert candidates(x, 2).tolist() == [1, 3]
    keys = ordered_keys(x)
    assert keys[4] == 0 and keys[5] > keys[2] > keys[6]
    assert greedy(x[[0, 1, 2, 3]]) == 1 and sample_ref(x, 0.0, 5, 123) == 1


def test_the_deterministic_exp2_is_close_and_exact_where_it_must_be():
    z = np.linspace(-60, 0, 4001).astype(np.float32)
    got = exp2_det(z).astype(np.float64)
    assert np.abs(got / np.exp2(z.astype(np.float64)) - 1).max() < 3e-7
    assert exp2_det(np.array([0, -1, -7, -120], np.float32)).tolist() == [1.0, 0.5, 2.0 ** -7, 2.0 ** -120]
    assert exp2_det(np.array([-121, -500, -np.inf, np.nan], np.float32)).tolist() == [0.0, 0.0, 0.0, 0.0]


def test_weights_follow_the_softmax_of_the_top_k():
    rng = np.random.default_rng(0)
    logits = (rng.standard_normal(4096) * 3).astype(bfloat16)
    for t, k in ((0.7, 50), (1.0, 8), (0.25, 64), (3.0, 1000)):
        cand, w = sample_weights(logits, t, k)
        kk = min(k, K_MAX)
        assert cand.size == kk and w[0] == 1.0
        top = np.sort(logits.astype(np.float64))[::-1][:kk]
        want = np.exp((top - top[0]) / np.float32(t))
        assert np.abs(w / want - 1).max() < 2e-6
        p = Sampler(t, k).probabilities(logits)
        assert abs(p.sum() - 1) < 1e-12 and np.count_nonzero(p) <= kk


def test_draws_cover_the_distribution_and_repeat_at_a_seed():
    logits = np.array([2.0, 1.0, 0.0, -1.0] + [-30.0] * 60, np.float32).astype(bfloat16)
    a, b = Sampler(1.0, 4, seed=7), Sampler(1.0, 4, seed=7)
    drawn = [a(logits) for _ in range(4000)]
    assert drawn[:50] == [b(logits) for _ in range(50)]
    freq = np.bincount(drawn, minlength=4)[:4] / 4000
    want = np.exp([2.0, 1, 0, -1]) / np.exp([2.0, 1, 0, -1]).sum()
    assert np.abs(freq - want).max() < 0.03 and max(drawn) < 4
    # the ends of the uniform: the first candidate at 0, the last at 2^53 - 1
    assert sample_ref(logits, 1.0, 4, 0) == 0 and sample_ref(logits, 1.0, 4, 2 ** 53 - 1) == 3
    assert sample_ref(np.full(16, 1.5, np.float32), 0.8, 4, 2 ** 52) == 2   # ties: lowest indices, equal weights


def test_rows_hold_what_the_host_draws_would_use():
    s, h = Sampler(0.7, 50, seed=3), Sampler(0.7, 50, seed=3)
    rows = s.rows(5)
    assert rows.shape == (5, ROW_WORDS) and rows.dtype == np.int32
    logits = (np.random.default_rng(1).standard_normal(512) * 2).astype(bfloat16)
    for row in rows:
        u = row.view(np.uint32)
        assert u[:1].view(np.float32)[0] == np.float32(0.7) and u[1] == 50
        assert sample_ref(logits, 0.7, 50, int(u[2]) | (int(u[3]) << 32)) == h(logits)
    assert not draw_row(0.0, 0, 0).any()
    with pytest.raises(ValueError, match="not one the device draws"):
        Sampler(0.7, None).rows(1)
    with pytest.raises(ValueError, match="not one the device draws"):
        Sampler(0.7, K_MAX + 1).rows(1)
    with pytest.raises(ValueError, match="negative"):
        Sampler(-1.0)
    with pytest.raises(ValueError, match="keeps no token"):
        Sampler(0.7, 0)
