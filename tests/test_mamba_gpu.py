"""Mamba2 selective scan and causal conv against the oracle (B200).

Scan cases are the reference's own (iron/operators/selective_scan.py:70-96) plus the
Granite-4.0-H layer shape (48 heads of 64, state 128, 3328 channels); the tolerance is the operator's,
``relative(8e-3, range_frac=1e-3)`` (selective_scan.py:353-356).
"""

import numpy as np
import pytest
from ml_dtypes import bfloat16

from iron_b200.verify import Tolerance
from oracle import ops
from tests.util import assert_verdict, normal, to_numpy, to_torch

pytestmark = pytest.mark.gpu
SCAN_TOL = Tolerance.relative(8e-3, range_frac=1e-3)


@pytest.fixture(scope="module")
def K():
    from iron_b200 import kernels

    return kernels


@pytest.fixture(params=["chunked, tensor memory", "chunked, warp MMAs", "step by step"])
def form(request):
    """The forms of the scan: prompt-length calls on the 64-wide-head shapes take a chunked
    tensor-core kernel unless it is switched off -- tcgen05 with 128-row chunks where there are 128
    states and 128 rows, warp MMAs with 64-row chunks otherwise -- everything else runs step by step."""
    from iron_b200 import _lib

    lib = _lib.load()
    mode = {"chunked, tensor memory": 2, "chunked, warp MMAs": 1, "step by step": 0}[request.param]
    lib.iron_set_scan_chunked(mode)
    yield "chunked" if mode else "step by step"
    lib.iron_set_scan_chunked(2)


def state_tolerance(form):
    """Both forms keep the state in float32; the chunked form adds a chunk's rows as a bf16 head
    and a bf16 remainder, which is float32's accuracy but another order of the sums."""
    return Tolerance.relative(2e-4 if form == "chunked" else 1e-4, atol=2e-4 if form == "chunked" else 1e-5)


def trained(rows, H, P, N, G, seed=3):
    """Heads as a trained Mamba2's are (selective_scan.py:32-43): A < 0, so the state decays."""
    rng = np.random.default_rng(seed)
    head = np.stack([rng.uniform(-4, 0, H), -rng.uniform(0.5, 16, H), rng.uniform(0, 2, H)], 1).astype(np.float32)
    xbc = (rng.standard_normal((rows, H * P + 2 * G * N)) * 0.5).astype(bfloat16)
    dt = normal(rng, (rows, H))
    state = rng.standard_normal((H, P, N), dtype=np.float32)
    return xbc, dt, head, state


SCAN_CASES = [
    # rows, heads, head_dim, state_size, groups
    (5, 2, 16, 16, 1), (8, 4, 32, 32, 2), (1, 2, 16, 128, 1), (3, 2, 16, 64, 1),
    (64, 16, 64, 64, 2), (2048, 8, 64, 16, 1), (300, 6, 64, 128, 1), (100, 4, 128, 32, 4),
    (128, 3, 64, 128, 1), (1000, 8, 64, 128, 2), (129, 2, 64, 128, 2),
]


@pytest.mark.parametrize("rows,H,P,N,G", SCAN_CASES)
def test_selective_scan_matches_reference(K, form, rows, H, P, N, G):
    xbc, dt, head, state = trained(rows, H, P, N, G)
    want_y, want_s = ops.selective_scan(xbc, dt, head, state, heads=H, head_dim=P, state_size=N, groups=G)
    y, final = K.selective_scan(to_torch(xbc), to_torch(dt), to_torch(head), to_torch(state),
                                heads=H, head_dim=P, state_size=N, groups=G)
    assert_verdict(to_numpy(y), want_y, SCAN_TOL, what="y")
    assert_verdict(to_numpy(final), want_s, state_tolerance(form), what="final state")


def test_scan_bounded_rows_and_chunked_equals_whole(K, form):
    import torch

    rows, H, P, N, G = 200, 4, 64, 128, 1
    xbc, dt, head, state = trained(rows, H, P, N, G, seed=5)
    want_y, want_s = ops.selective_scan(xbc, dt, head, state, heads=H, head_dim=P, state_size=N, valid=131)
    nv = torch.tensor([131], dtype=torch.int32, device="cuda")
    y, final = K.selective_scan(to_torch(xbc), to_torch(dt), to_torch(head), to_torch(state), heads=H,
                                head_dim=P, state_size=N, d_valid=nv)
    got = to_numpy(y)
    assert_verdict(got, want_y, SCAN_TOL)
    assert not got[131:].astype(np.float32).any()
    assert_verdict(to_numpy(final), want_s, state_tolerance(form))
    # two calls, the second starting from the first's final state, equal one call
    y1, mid = K.selective_scan(to_torch(xbc[:77]), to_torch(dt[:77]), to_torch(head), to_torch(state),
                               heads=H, head_dim=P, state_size=N)
    y2, end = K.selective_scan(to_torch(xbc[77:]), to_torch(dt[77:]), to_torch(head), mid, heads=H,
                               head_dim=P, state_size=N)
    whole, end_whole = K.selective_scan(to_torch(xbc), to_torch(dt), to_torch(head), to_torch(state),
                                        heads=H, head_dim=P, state_size=N)
    if form == "chunked":   # 77 + 123 rows cut the 64-row chunks elsewhere than 200 rows do
        assert_verdict(to_numpy(torch.cat([y1, y2])), to_numpy(whole), SCAN_TOL)
        assert_verdict(to_numpy(end), to_numpy(end_whole), state_tolerance(form))
    else:
        assert torch.equal(torch.cat([y1, y2]), whole) and torch.allclose(end, end_whole, rtol=1e-5, atol=1e-6)


def test_granite_hybrid_layer_shape_batched(K, form):
    """d_inner 3072 = 48 heads x 64, d_state 128, 1 group; batch 2 x 512 rows of the 8 x 4096 config."""
    rng = np.random.default_rng(5001)
    B, rows, H, P, N = 2, 512, 48, 64, 128
    xbc = normal(rng, (B, rows, H * P + 2 * N))
    dt = (rng.standard_normal((B, rows, H), dtype=np.float32) - 4).astype(bfloat16)
    head = np.stack([np.zeros(H), -np.exp(rng.uniform(0, 2.7, H)), np.ones(H)], 1).astype(np.float32)
    y, final = K.selective_scan(to_torch(xbc), to_torch(dt), to_torch(head), None, heads=H, head_dim=P,
                                state_size=N)
    for b in range(B):
        want_y, want_s = ops.selective_scan(xbc[b], dt[b], head, np.zeros((H, P, N), np.float32), heads=H,
                                            head_dim=P, state_size=N)
        assert_verdict(to_numpy(y[b]), want_y, SCAN_TOL, what=f"y[{b}]")
        assert_verdict(to_numpy(final[b]), want_s, state_tolerance(form))


@pytest.mark.parametrize("rows,C,Kt,decode", [(1, 3328, 4, True), (300, 3328, 4, False), (2048, 256, 4, False),
                                               (17, 64, 2, False), (5, 128, 3, False)])
def test_causal_conv_is_bit_exact_with_the_recorded_chain(K, rows, C, Kt, decode):
    rng = np.random.default_rng(11)
    x, taps = normal(rng, (rows, C)), normal(rng, (Kt, C), 0.5)
    hist, bias = normal(rng, (Kt - 1, C)), normal(rng, (C,), 0.1)
    if decode:
        # the one-row form sums the newest tap first (iron/functional.py:166-170)
        full = np.concatenate([hist, x])
        want = ops.mul(x, taps[Kt - 1])
        for k in range(Kt - 1):
            want = ops.add(want, ops.mul(full[k : k + 1], taps[k]))
        new_hist = full[1:]
    else:
        want, new_hist = ops.causal_conv1d(x, taps, hist)
    want = ops.silu(ops.add(want, bias))
    import torch

    nh = torch.empty((Kt - 1, C), dtype=torch.bfloat16, device="cuda")
    got = to_numpy(K.causal_conv1d(to_torch(x), to_torch(taps), bias=to_torch(bias), history=to_torch(hist),
                                   new_history=nh, decode_order=decode, silu=True))
    assert_verdict(got, want, Tolerance.bf16_ulps(1), what="conv + bias + silu")
    assert np.array_equal(to_numpy(nh).view(np.uint16), new_hist.view(np.uint16))
    # without the activation the chain is exact
    got = to_numpy(K.causal_conv1d(to_torch(x), to_torch(taps), history=to_torch(hist), decode_order=decode))
    plain = want_plain(x, taps, hist, decode)
    assert np.array_equal(got.view(np.uint16), plain.view(np.uint16))


def want_plain(x, taps, hist, decode):
    Kt = taps.shape[0]
    if not decode:
        return ops.causal_conv1d(x, taps, hist)[0]
    full = np.concatenate([hist, x])
    want = ops.mul(x, taps[Kt - 1])
    for k in range(Kt - 1):
        want = ops.add(want, ops.mul(full[k : k + 1], taps[k]))
    return want


def mixer_weights(E, H, P, N, G, Kc, seed):
    """A mixer's checkpoint tensors: projections N(0, 1/sqrt(in)), taps N(0, 1/2), decays and
    time steps as Mamba2 initialises them (A = -exp(U(0, 2.7)), softplus^-1 of dt in 1e-3..1e-1)."""
    rng = np.random.default_rng(seed)
    inner, C = H * P, H * P + 2 * G * N
    dt = np.exp(rng.uniform(np.log(1e-3), np.log(1e-1), H))
    return {
        "in_proj.weight": normal(rng, (inner + C + H, E), 1 / np.sqrt(E)),
        "conv1d.weight": normal(rng, (C, 1, Kc), 0.5),
        "conv1d.bias": normal(rng, (C,), 0.1),
        "dt_bias": (dt + np.log(-np.expm1(-dt))).astype(bfloat16),
        "A_log": rng.uniform(0, 2.7, H).astype(bfloat16),
        "D": np.ones(H, bfloat16),
        "norm.weight": (1 + rng.standard_normal(inner) / 10).astype(bfloat16),
        "out_proj.weight": normal(rng, (E, inner), 1 / np.sqrt(inner)),
    }


def assert_layer_close(got, want, what):
    """The mixer's output is a 3072-term projection of normed rows: a one-ulp flip in the scan's
    bf16 output moves it by an amount set by the output's scale, so the bound is 2 % of the
    largest output (each kernel alone is held to its operator's tolerance above)."""
    got, want = np.asarray(got, np.float32), np.asarray(want, np.float32)
    err = np.abs(got - want).max()
    assert err <= 0.02 * np.abs(want).max(), f"{what}: max error {err:.4g} against {np.abs(want).max():.4g}"


def test_the_fused_mixer_matches_the_oracle_mixer_across_calls():
    """Two sequences, a chunk of 200 rows, a chunk of 57 and three decode steps: the
    convolution rows and scan states carry from call to call, per sequence."""
    from iron_b200.lm.mamba import MambaMixer
    from oracle import model as M

    E, H, P, N, G, Kc = 256, 8, 64, 64, 2, 4
    w = mixer_weights(E, H, P, N, G, Kc, 41)
    mixer = MambaMixer(w, hidden_size=E, heads=H, head_dim=P, state_size=N, groups=G, kernel=Kc, eps=1e-6,
                       batch=2, rows=256)
    rng = np.random.default_rng(42)
    C = H * P + 2 * G * N
    states = [(np.zeros((Kc - 1, C), bfloat16), np.zeros((H, P, N), np.float32)) for _ in range(2)]
    for rows in (200, 57, 1, 1, 1):
        x = normal(rng, (2, rows, E))
        got = to_numpy(mixer.forward(to_torch(x)))
        for b in range(2):
            want, conv, ssm = M.mamba_mixer(x[b], w, "", *states[b], heads=H, head_dim=P, state_size=N,
                                            groups=G, kernel=Kc, eps=1e-6)
            states[b] = (conv, ssm)
            assert_layer_close(got[b], want, f"sequence {b}, {rows} rows")
    mixer.check()


def test_one_sequence_of_the_full_layer_shape_at_4096_rows(K):
    """d_model 1536 -> d_inner 3072 (48 heads of 64), state 128, one group, 4096 rows: one batch
    entry of the 8 x 4096 layer, the scan alone against the sequential oracle and the whole
    mixer against the oracle mixer."""
    from iron_b200.lm.mamba import MambaMixer
    from oracle import model as M

    E, H, P, N, G, Kc, rows = 1536, 48, 64, 128, 1, 4, 4096
    rng = np.random.default_rng(5001)
    xbc = normal(rng, (rows, H * P + 2 * N))
    dt = (rng.standard_normal((rows, H), dtype=np.float32) - 4).astype(bfloat16)
    head = np.stack([np.zeros(H), -np.exp(rng.uniform(0, 2.7, H)), np.ones(H)], 1).astype(np.float32)
    want_y, want_s = ops.selective_scan(xbc, dt, head, np.zeros((H, P, N), np.float32), heads=H, head_dim=P,
                                        state_size=N)
    y, final = K.selective_scan(to_torch(xbc), to_torch(dt), to_torch(head), None, heads=H, head_dim=P,
                                state_size=N)
    assert_verdict(to_numpy(y), want_y, SCAN_TOL, what="scan, 4096 rows")
    assert_verdict(to_numpy(final), want_s, Tolerance.relative(1e-4, atol=1e-4), what="final state")
    w = mixer_weights(E, H, P, N, G, Kc, 43)
    mixer = MambaMixer(w, hidden_size=E, heads=H, head_dim=P, state_size=N, groups=G, kernel=Kc, batch=1,
                       rows=rows)
    x = normal(rng, (1, rows, E))
    got = to_numpy(mixer.forward(to_torch(x)))[0]
    want, _, _ = M.mamba_mixer(x[0], w, "", np.zeros((Kc - 1, H * P + 2 * N), bfloat16),
                               np.zeros((H, P, N), np.float32), heads=H, head_dim=P, state_size=N, groups=G,
                               kernel=Kc)
    assert_layer_close(got, want, "mixer, 4096 rows")
    mixer.check()
