"""Prompt-chunk attention against the oracle's MHA reference (B200).

Cases follow iron/operators/mha.py:78-174 (chunk over a cache, grouped-query heads,
windows, bidirectional) and the bounded-row rule of
iron/tests/operators/test_mha_bounded_rows.py:99-111.
"""

import numpy as np
import pytest

from iron_b200.verify import Tolerance
from oracle import ops
from tests.util import assert_verdict, normal, to_numpy, to_torch

pytestmark = pytest.mark.gpu
MHA_TOL = Tolerance(rtol=0.04, atol=0.15, max_mismatch_frac=0.005)  # mha.py:1118-1126
TIGHT = Tolerance.relative(0.02, atol=2e-2)


@pytest.fixture(scope="module")
def K():
    from iron_b200 import kernels

    return kernels


CASES = [
    # H, G, D, q_rows, kv_rows, q_tokens, kv_tokens, causal, window
    (8, 2, 64, 256, 256, None, None, True, None),
    (8, 2, 64, 512, 2048, None, None, True, None),      # a chunk over a cache
    (32, 8, 64, 2048, 2048, None, None, True, None),    # Llama 1B's first prompt chunk
    (24, 8, 128, 512, 1024, None, None, True, None),    # Llama 3B's head shape
    (4, 1, 64, 200, 300, 130, 270, True, None),         # ragged bounds
    (4, 2, 64, 128, 512, 77, 77, True, None),           # a short prompt in a long cache
    (4, 1, 64, 512, 2048, None, None, True, 511),       # sliding window
    (4, 2, 64, 320, 320, None, None, False, 100),       # bidirectional window
    (4, 1, 128, 192, 192, None, None, False, None),     # bidirectional, all keys
    (2, 2, 64, 64, 64, 1, 1, True, None),               # one token
]


@pytest.mark.parametrize("H,G,D,qr,kr,qt,kt,causal,window", CASES)
def test_prefill_attention_matches_reference(K, H, G, D, qr, kr, qt, kt, causal, window):
    rng = np.random.default_rng(42)
    q, k, v = normal(rng, (qr, H, D)), normal(rng, (kr, G, D)), normal(rng, (kr, G, D))
    want = ops.mha(q, k, v, num_heads=H, num_kv_heads=G, causal=causal, window=window,
                   heads_interleaved=True, kv_interleaved=True, q_tokens=qt, kv_tokens=kt)
    got = to_numpy(K.mha_prefill(to_torch(q), to_torch(k), to_torch(v), q_tokens=qt, kv_tokens=kt,
                                 causal=causal, window=window))
    assert_verdict(got, want, MHA_TOL, what="prefill attention")
    assert_verdict(got, want, TIGHT, what="prefill attention (tight)")
    if qt is not None:
        assert not got[qt:].astype(np.float32).any(), "rows past the bound must be exactly zero"
    assert not np.isnan(got.astype(np.float32)).any()


def test_bounds_from_device_values_and_head_major_layout(K):
    import torch

    rng = np.random.default_rng(3)
    H, G, D, S = 8, 4, 64, 256
    q, k, v = normal(rng, (H, S, D)), normal(rng, (G, S, D)), normal(rng, (G, S, D))
    want = ops.mha(q, k, v, num_heads=H, num_kv_heads=G, q_tokens=100, kv_tokens=180)
    nq = torch.tensor([100], dtype=torch.int32, device="cuda")
    pos = torch.tensor([179], dtype=torch.int32, device="cuda")
    got = to_numpy(K.mha_prefill(to_torch(q), to_torch(k), to_torch(v), d_q_tokens=nq, d_kv_tokens=pos,
                                 kv_tokens_add=1, heads_interleaved=False, kv_interleaved=False))
    assert_verdict(got, want, TIGHT)
    assert not got[:, 100:].astype(np.float32).any()


@pytest.mark.parametrize("H,G,D,qr,kr,qt,kt,causal,window", [c for c in CASES if (c[5] or c[3]) >= 128])
def test_the_tensor_memory_kernel_and_the_warp_mma_kernel_agree(K, monkeypatch, H, G, D, qr, kr, qt, kt, causal, window):
    """Calls with host-known bounds and at least 128 queries take the tcgen05 kernel; the same
    call with it switched off takes the warp-MMA kernel.  Same arithmetic, other summation
    order: the outputs agree to a bf16 rounding of values of order one."""
    rng = np.random.default_rng(11)
    q, k, v = (to_torch(normal(rng, s)) for s in ((qr, H, D), (kr, G, D), (kr, G, D)))
    out = {}
    for mode in ("1", "0"):
        monkeypatch.setenv("IRON_MHA_PREFILL_TC", mode)
        out[mode] = to_numpy(K.mha_prefill(q, k, v, q_tokens=qt, kv_tokens=kt, causal=causal,
                                           window=window)).astype(np.float32)
    assert np.abs(out["1"] - out["0"]).max() <= 2 ** -6
    assert int(K.prefill_status().item()) == 0


def test_the_tensor_memory_kernel_on_batches_head_major_layouts_and_strided_queries(K):
    import torch

    rng = np.random.default_rng(5)
    B, H, G, D, S = 3, 8, 4, 64, 384
    q, k, v = normal(rng, (B, H, S, D)), normal(rng, (B, G, S, D)), normal(rng, (B, G, S, D))
    got = to_numpy(K.mha_prefill(to_torch(q), to_torch(k), to_torch(v), q_tokens=300, kv_tokens=300,
                                 heads_interleaved=False, kv_interleaved=False))
    for b in range(B):
        want = ops.mha(q[b], k[b], v[b], num_heads=H, num_kv_heads=G, q_tokens=300, kv_tokens=300)
        assert_verdict(got[b], want, TIGHT, what=f"batch {b}")
        assert not got[b][:, 300:].astype(np.float32).any()
    # queries as a strided view of a fused q/k/v projection, the way the prompt path calls it
    n, Hq, Gk = 256, 8, 2
    qkv = normal(rng, (n, (Hq + 2 * Gk) * D))
    kc, vc = normal(rng, (512, Gk, D)), normal(rng, (512, Gk, D))
    t = to_torch(qkv)
    got = to_numpy(K.mha_prefill(t.view(n, Hq + 2 * Gk, D)[:, :Hq], to_torch(kc), to_torch(vc),
                                 torch.empty(n, Hq, D, dtype=torch.bfloat16, device="cuda"),
                                 q_tokens=n, kv_tokens=400, q_row_stride=t.stride(0)))
    want = ops.mha(qkv.reshape(n, Hq + 2 * Gk, D)[:, :Hq], kc, vc, num_heads=Hq, num_kv_heads=Gk,
                   heads_interleaved=True, kv_interleaved=True, q_tokens=n, kv_tokens=400)
    assert_verdict(got, want, TIGHT, what="strided queries over a cache")
    assert int(K.prefill_status().item()) == 0


def test_long_context_decode_accuracy_deep_in_the_cache(K):
    """iron/tests/operators/test_mha_long_context.py:45-62: one query at positions 1023 and
    32703 stays within 4 % of the output range."""
    rng = np.random.default_rng(8)
    H, G, D, S = 32, 8, 64, 32768
    k, v = normal(rng, (S, G, D)), normal(rng, (S, G, D))
    for pos in (1023, 32703):
        q = normal(rng, (1, H, D))
        want = ops.mha(q, k, v, num_heads=H, num_kv_heads=G, heads_interleaved=True,
                       kv_interleaved=True, q_tokens=1, kv_tokens=pos + 1).astype(np.float32)
        ns = None
        got = to_numpy(K.mha_decode(to_torch(q), to_torch(k), to_torch(v), kv_valid=pos + 1, nsplit=ns)).astype(np.float32)
        assert np.abs(got - want).max() <= 0.04 * (want.max() - want.min())
