"""The device draw against the host sampler: the same token from the same logits and uniform (B200)."""

import numpy as np
import pytest
from ml_dtypes import bfloat16

from iron_b200.lm.generation import ROW_WORDS, Sampler, draw_row, sample_ref
from tests.util import to_torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def K():
    from iron_b200 import kernels

    return kernels


def device_draws(K, logits, rows_of_draws, positions, S):
    """Run the kernel on ``logits`` (rows, n) with one draw row per row at its position."""
    import torch

    rows = logits.shape[0]
    draws = np.zeros((rows, S, ROW_WORDS), np.int32)
    for r in range(rows):
        draws[r, positions[r]] = rows_of_draws[r]
    tokens = torch.full((rows,), -1, dtype=torch.int32, device="cuda")
    pos = torch.tensor(positions, dtype=torch.int32, device="cuda")
    drawn = torch.full((rows, S), -1, dtype=torch.int32, device="cuda")
    K.sample_rows(to_torch(logits), torch.from_numpy(draws).cuda(), tokens, pos, drawn)
    return tokens.cpu().numpy(), pos.cpu().numpy(), drawn.cpu().numpy()


@pytest.mark.parametrize("n,t,k", [(1024, 0.7, 50), (128256, 0.7, 50), (128256, 1.0, 64), (4099, 0.3, 7),
                                   (50000, 2.5, 64), (64, 1.0, 64), (40, 0.9, 64), (128256, 0.7, 2)])
def test_the_device_picks_the_host_samplers_token(K, n, t, k):
    rng = np.random.default_rng(n + k)
    rows, S = 24, 8
    logits = (rng.standard_normal((rows, n)) * 3).astype(bfloat16)
    n53 = [int(rng.integers(0, 2 ** 53)) for _ in range(rows)]
    n53[0], n53[1] = 0, 2 ** 53 - 1                      # the ends of the uniform
    positions = [int(rng.integers(0, S)) for _ in range(rows)]
    got, pos_after, drawn = device_draws(K, logits, [draw_row(t, k, u) for u in n53], positions, S)
    want = [sample_ref(logits[r], t, k, n53[r]) for r in range(rows)]
    assert got.tolist() == want
    assert pos_after.tolist() == [p + 1 for p in positions]
    for r in range(rows):
        assert drawn[r, positions[r]] == want[r] and (np.delete(drawn[r], positions[r]) == -1).all()


def test_ties_special_values_and_greedy_rows(K):
    rng = np.random.default_rng(5)
    n, S = 8192, 4
    base = (rng.standard_normal(n) * 2).astype(np.float32)
    cases = []
    flat = np.full(n, 1.5, np.float32)                   # every logit equal: the lowest indices, equal weights
    cases.append(flat)
    plateau = base.copy(); plateau[rng.choice(n, 300, replace=False)] = 9.0   # more ties at the top than k
    cases.append(plateau)
    edge = base.copy(); edge[:40] = 7.0; edge[100:130] = 6.5                  # the threshold falls inside a tie
    cases.append(edge)
    special = base.copy(); special[3] = np.nan; special[4] = np.inf; special[5] = -np.inf; special[6] = -0.0
    cases.append(special)
    neg = -np.abs(base) - 50.0                           # all negative, far from zero
    cases.append(neg)
    logits = np.stack(cases).astype(bfloat16)
    for t, k in ((0.8, 50), (1.3, 64), (0.5, 3)):
        n53 = [int(rng.integers(0, 2 ** 53)) for _ in cases]
        got, _, _ = device_draws(K, logits, [draw_row(t, k, u) for u in n53], [1] * len(cases), S)
        assert got.tolist() == [sample_ref(logits[r], t, k, n53[r]) for r in range(len(cases))]
    # all-zero rows, temperature 0 and top_k 1 are the greedy draw: the first index of the maximum
    greedy_rows = [np.zeros(ROW_WORDS, np.int32), draw_row(0.0, 50, 12345), draw_row(0.7, 1, 999), draw_row(0.7, 50, 7),
                   draw_row(0.7, 50, 8)]
    got, _, _ = device_draws(K, logits, greedy_rows, [0] * len(cases), S)
    first_max = [int(np.argmax(logits[r].astype(np.float32))) for r in range(3)]
    assert got[:3].tolist() == first_max and first_max[0] == 0
    assert got[3] == sample_ref(logits[3], 0.7, 50, 7) and got[4] == sample_ref(logits[4], 0.7, 50, 8)


def test_a_sampler_stream_matches_draw_for_draw(K):
    """``Sampler.rows`` gives the device the uniforms the host draws would use, in order."""
    rng = np.random.default_rng(9)
    n, S = 32000, 16
    logits = (rng.standard_normal((1, n)) * 4).astype(bfloat16)
    device, host = Sampler(0.7, 50, seed=11), Sampler(0.7, 50, seed=11)
    rows = device.rows(S)
    for p in range(S):
        got, _, _ = device_draws(K, logits, [rows[p]], [p], S)
        assert int(got[0]) == host(logits[0])
