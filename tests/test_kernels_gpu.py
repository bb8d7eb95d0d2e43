"""Parity of the bandwidth-bound kernels with the CPU oracle, through the C ABI (B200).

Shapes follow the reference's own case lists (iron/operators/gemv.py:24-76,
rope.py:24-55, mha.py:78-174) plus the 1B decode-chain sizes; tolerances are each
operator's own ``tolerance()`` and the bf16 output bound (1e-2 relative / 2e-2 absolute),
exact for integer and data-movement results.
"""

import numpy as np
import pytest
from ml_dtypes import bfloat16

from iron_b200.verify import Tolerance
from oracle import ops
from oracle.model import rope_angles
from tests.util import assert_bf16_bound, assert_verdict, normal, to_numpy, to_torch

pytestmark = pytest.mark.gpu

GEMV_TOL = Tolerance.relative(0.04, 1e-3)   # iron/operators/gemv.py:419-421
ROPE_TOL = Tolerance.relative(0.05)         # iron/operators/rope.py:186-191
MHA_TOL = Tolerance(rtol=0.04, atol=0.15, max_mismatch_frac=0.005)  # mha.py:1118-1126


@pytest.fixture(scope="module")
def K():
    from iron_b200 import kernels

    return kernels


# M, K, num_batches, repeat -- the reference's plain, batched and repeated cases
GEMV_CASES = [
    (128, 128, None, 1), (2048, 8192, None, 1), (8192, 2048, None, 1), (1536, 12288, None, 1),
    (256, 128, 4, 1), (256, 128, 100, 1), (448, 64, 192, 1), (64, 1536, 8, 1),
    (1026, 64, 2, 1), (1024, 1024, 2, 1), (512, 64, 32, 1),
    (256, 128, 8, 4), (256, 128, 4, 4), (1024, 1024, 4, 2), (2048, 64, 32, 4),
    (3072, 2048, None, 1), (2047, 2048, None, 1), (33, 72, None, 1),
]


@pytest.mark.parametrize("M,Kd,batches,repeat", GEMV_CASES)
def test_gemv_matches_reference(K, M, Kd, batches, repeat):
    rng = np.random.default_rng(42)
    if batches is None:
        A, B = normal(rng, (M, Kd)), normal(rng, (Kd,))
    else:
        A, B = normal(rng, (batches // repeat, M, Kd)), normal(rng, (batches, Kd))
    want = ops.gemv(A, B, repeat)
    got = to_numpy(K.gemv(to_torch(A), to_torch(B), repeat=repeat))
    assert_verdict(got, want, GEMV_TOL, what=f"GEMV {M}x{Kd} b={batches} r={repeat}")


def test_gemv_bounded_rows_leave_the_rest_untouched(K):
    rng = np.random.default_rng(1)
    A, B = normal(rng, (256, 512)), normal(rng, (512,))
    import torch

    out = torch.full((256,), 7.0, dtype=torch.bfloat16, device="cuda")
    K.gemv(to_torch(A), to_torch(B), out, valid=101)
    got = to_numpy(out)
    assert_verdict(got[:101], ops.gemv(A, B)[:101], GEMV_TOL)
    assert (got[101:].astype(np.float32) == 7.0).all()


@pytest.mark.parametrize("weighted", [False, True])
def test_gemv_with_fused_rmsnorm_and_residual(K, weighted):
    rng = np.random.default_rng(2001)
    x = normal(rng, (2048,))
    w = (1 + rng.standard_normal(2048, dtype=np.float32) * 0.02).astype(bfloat16)
    W = normal(rng, (2048, 2048), 0.02)
    res = normal(rng, (2048,))
    h = ops.rms_norm(x, w if weighted else None, 1e-5)
    want = ops.add(res, ops.gemv(W, h))
    got = to_numpy(K.gemv(to_torch(W), to_torch(x), norm_weight=to_torch(w) if weighted else None,
                          norm=True, eps=1e-5, residual=to_torch(res)))
    assert_verdict(got, want, GEMV_TOL)
    assert_bf16_bound(got, want, "norm+gemv+residual")


def test_gate_up_swiglu_matches_the_unfused_chain(K):
    rng = np.random.default_rng(2004)
    x = normal(rng, (2048,))
    w = (1 + rng.standard_normal(2048, dtype=np.float32) * 0.02).astype(bfloat16)
    Wg, Wu = normal(rng, (8192, 2048), 0.02), normal(rng, (8192, 2048), 0.02)
    h = ops.rms_norm(x, w, 1e-5)
    want = ops.mul(ops.silu(ops.gemv(Wg, h)), ops.gemv(Wu, h))
    got = to_numpy(K.gemv_swiglu(to_torch(Wg), to_torch(Wu), to_torch(x), norm_weight=to_torch(w)))
    assert_verdict(got, want, GEMV_TOL)
    assert_bf16_bound(got, want, "swiglu")


@pytest.mark.parametrize("H,G,D,E", [(32, 8, 64, 2048), (24, 8, 128, 3072)])
def test_decode_qkv_rope_writes_q_and_the_cache_row(K, H, G, D, E):
    import torch

    rng = np.random.default_rng(2002)
    pos, S = 1023, 1100
    x = normal(rng, (E,))
    w = (1 + rng.standard_normal(E, dtype=np.float32) * 0.02).astype(bfloat16)
    W = normal(rng, ((H + 2 * G) * D, E), 0.02)
    table = rope_angles(D, S, 500000.0).astype(bfloat16)
    h = ops.rms_norm(x, w, 1e-5)
    qkv = ops.gemv(W, h)
    q = ops.rope(qkv[: H * D].reshape(H, D), table[pos : pos + 1])
    k = ops.rope(qkv[H * D : (H + G) * D].reshape(G, D), table[pos : pos + 1])
    v = qkv[(H + G) * D :].reshape(G, D)
    kc = torch.zeros((S, G, D), dtype=torch.bfloat16, device="cuda")
    vc = torch.zeros_like(kc)
    qo = torch.empty((H, D), dtype=torch.bfloat16, device="cuda")
    dpos = torch.tensor([pos], dtype=torch.int32, device="cuda")
    K.decode_qkv_rope(to_torch(W), to_torch(x), to_torch(table), kc, vc, qo, H=H, G=G, D=D,
                      d_position=dpos, norm_weight=to_torch(w))
    assert_verdict(to_numpy(qo), q, ROPE_TOL, what="q")
    assert_verdict(to_numpy(kc[pos]), k, ROPE_TOL, what="k")
    assert_verdict(to_numpy(vc[pos]), v, GEMV_TOL, what="v")
    assert_bf16_bound(to_numpy(qo), q, "q")
    kc[pos] = 0
    vc[pos] = 0
    assert not kc.any() and not vc.any(), "only row `position` of the caches is written"


@pytest.mark.parametrize("rows,cols,weighted", [(1, 2048, True), (1, 3072, True), (7, 512, False),
                                                 (300, 4096, True), (2048, 2048, True)])
def test_rmsnorm(K, rows, cols, weighted):
    rng = np.random.default_rng(7)
    x = normal(rng, (rows, cols))
    w = (1 + rng.standard_normal(cols, dtype=np.float32) / 10).astype(bfloat16)
    want = ops.rms_norm(x, w if weighted else None, 1e-5)
    got = to_numpy(K.rms_norm(to_torch(x), to_torch(w) if weighted else None, eps=1e-5))
    assert_verdict(got, want, Tolerance.bf16_ulps(1), what="rmsnorm")


@pytest.mark.parametrize("rows,cols", [(5, 3072), (3, 64), (300, 8192), (2, 1032)])
def test_rmsnorm_of_a_gated_product_is_the_three_steps_in_one(K, rows, cols):
    """x * silu(gate), then RMSNorm: each of the three recorded steps rounds to bf16."""
    rng = np.random.default_rng(rows + cols)
    x, gate, w = normal(rng, (rows, cols), 2.0), normal(rng, (rows, cols), 2.0), normal(rng, (cols,))
    want = ops.rms_norm(ops.mul(x, ops.silu(gate)), w, 1e-5)
    got = to_numpy(K.rms_norm_gated(to_torch(x), to_torch(gate), to_torch(w), eps=1e-5))
    assert_verdict(got, want, Tolerance.bf16_ulps(2), what="gated rmsnorm")
    with pytest.raises(Exception):
        K.rms_norm_gated(to_torch(normal(rng, (2, 8200))), to_torch(normal(rng, (2, 8200))))


@pytest.mark.parametrize("rows,cols,angle_rows,two_halves", [
    (32, 512, 8, True), (32, 512, 32, True), (32, 128, 8, False), (64, 128, 16, True),
    (4096, 512, 8, True), (40, 64, 1, True), (2048 * 8, 64, 2048, True)])
def test_rope_is_bit_exact(K, rows, cols, angle_rows, two_halves):
    rng = np.random.default_rng(0)
    theta = rng.uniform(-np.pi, np.pi, (angle_rows, cols // 2))
    table = np.empty((angle_rows, cols), np.float32)
    table[:, ::2], table[:, 1::2] = np.cos(theta), np.sin(theta)
    table = table.astype(bfloat16)
    x = normal(rng, (rows, cols), 4.0)
    want = ops.rope(x, table, two_halves)
    got = to_numpy(K.rope(to_torch(x), to_torch(table), two_halves=two_halves))
    assert np.array_equal(got.view(np.uint16), want.view(np.uint16))


def test_rope_offset_and_bound_from_device_values(K):
    import torch

    rng = np.random.default_rng(5)
    table = rope_angles(64, 256).astype(bfloat16)
    x = normal(rng, (8 * 4, 64))
    out = torch.zeros((32, 64), dtype=torch.bfloat16, device="cuda")
    off = torch.tensor([100], dtype=torch.int32, device="cuda")
    nv = torch.tensor([20], dtype=torch.int32, device="cuda")
    K.rope(to_torch(x), to_torch(table), out, angle_rows=8, d_angle_offset=off, d_valid=nv)
    want = ops.rope(x, table[100:108])
    got = to_numpy(out)
    assert np.array_equal(got[:20].view(np.uint16), want[:20].view(np.uint16))
    assert not got[20:].astype(np.float32).any()


@pytest.mark.parametrize("n", [8192, 2048 * 8192 // 16, 1000, 13])
def test_elementwise_family(K, n):
    rng = np.random.default_rng(11)
    a, b = normal(rng, (n,), 2.0), normal(rng, (n,), 2.0)
    ta, tb = to_torch(a), to_torch(b)
    exact = lambda g, w: np.array_equal(to_numpy(g).view(np.uint16), w.view(np.uint16))
    assert exact(K.elementwise("add", ta, tb), ops.add(a, b))
    assert exact(K.elementwise("mul", ta, tb), ops.mul(a, b))
    assert exact(K.elementwise("axpy", ta, tb, scalar=1.003), ops.axpy(a, b, 1.003))
    assert_verdict(to_numpy(K.elementwise("silu", ta)), ops.silu(a), Tolerance.bf16_ulps(1))
    assert_verdict(to_numpy(K.elementwise("silu_mul", ta, tb)), ops.mul(ops.silu(a), b),
                   Tolerance.bf16_ulps(2, atol=1e-6))


def test_rowwise_broadcast(K):
    rng = np.random.default_rng(12)
    a, row = normal(rng, (64, 3328)), normal(rng, (3328,))
    exact = lambda g, w: np.array_equal(to_numpy(g).view(np.uint16), w.view(np.uint16))
    assert exact(K.elementwise("row_mul", to_torch(a), to_torch(row)), ops.mul(a, row))
    assert exact(K.elementwise("row_add", to_torch(a), to_torch(row)), ops.add(a, row))


def test_gather_and_strided_copy_are_exact(K):
    import torch

    rng = np.random.default_rng(13)
    table = normal(rng, (1000, 256))
    ids = np.array([5, 999, 0, 1500, -3, 17], np.int32)   # out-of-range ids clip
    out = torch.zeros((6, 256), dtype=torch.bfloat16, device="cuda")
    K.copy_rows(to_torch(table), out, ids=to_torch(ids), nrows=6, row_bytes=512, src_rows=1000)
    assert np.array_equal(to_numpy(out).view(np.uint16), ops.gather_rows(table, ids).view(np.uint16))
    # a run written at a per-call row of a cache, bounded per call
    cache = torch.zeros((64, 8, 64), dtype=torch.bfloat16, device="cuda")
    rows = normal(rng, (16, 8, 64))
    start = torch.tensor([40], dtype=torch.int32, device="cuda")
    n = torch.tensor([9], dtype=torch.int32, device="cuda")
    K.copy_rows(to_torch(rows), cache, nrows=16, row_bytes=1024, d_dst_row0=start, d_nrows=n)
    got = to_numpy(cache)
    assert np.array_equal(got[40:49].view(np.uint16), rows[:9].view(np.uint16))
    got[40:49] = 0
    assert not got.astype(np.float32).any()


@pytest.mark.parametrize("n", [128256, 1024, 77, 8])
def test_argmax_is_first_maximum(K, n):
    import torch

    rng = np.random.default_rng(n)
    logits = normal(rng, (n,), 3.0)
    hi = logits.astype(np.float32).max()
    # plant ties of the maximum: the first must win
    for i in rng.integers(0, n, 3):
        logits[i] = hi
    ws = K.argmax_workspace("cuda")
    tok = torch.zeros(1, dtype=torch.int32, device="cuda")
    carry = torch.zeros(2, dtype=torch.int32, device="cuda")
    carry[1] = 41
    for _ in range(2):  # the workspace is left ready for the next launch
        K.argmax(to_torch(logits), tok, ws, carry_token=carry[0:1], carry_position=carry[1:2])
        assert int(tok.item()) == ops.greedy(logits)
    assert carry.tolist() == [ops.greedy(logits), 43]


MHA_DECODE_CASES = [
    # H, G, D, kv_len, kv_valid, window, nsplit
    (32, 8, 64, 2048, 2048, None, 8),
    (32, 8, 64, 2048, 1024, None, 4),
    (32, 8, 64, 2048, 1, None, 4),
    (32, 8, 64, 2048, 77, None, 1),
    (40, 8, 64, 2048, 2048, None, 8),
    (24, 8, 128, 2048, 2000, None, 8),
    (4, 1, 256, 2048, 2048, 511, 8),
    (8, 2, 64, 512, 512, None, 2),
    (8, 8, 64, 300, 300, None, None),
    (16, 1, 64, 256, 200, None, 2),
    (32, 8, 64, 8192, 8000, None, 8),
]


@pytest.mark.parametrize("H,G,D,S,n,window,nsplit", MHA_DECODE_CASES)
def test_mha_decode_matches_reference(K, H, G, D, S, n, window, nsplit):
    rng = np.random.default_rng(42)
    q = normal(rng, (1, H, D))
    k, v = normal(rng, (S, G, D)), normal(rng, (S, G, D))
    want = ops.mha(q, k, v, num_heads=H, num_kv_heads=G, window=window, heads_interleaved=True,
                   kv_interleaved=True, q_tokens=1, kv_tokens=n)
    ns = nsplit
    tq, tk, tv = to_torch(q), to_torch(k), to_torch(v)
    # twice each (the resident form's arrival counters must be back at zero), and with the promise that only
    # the newest row is fresh (its keys are then asked for ahead of the dependency wait, that row after it)
    for stable in (False, True, False, True):
        got = to_numpy(K.mha_decode(tq, tk, tv, kv_valid=n, window=window, nsplit=ns, stable_prefix=stable))
        assert_verdict(got, want, MHA_TOL, what=f"mha decode, stable_prefix={stable}")
        assert_bf16_bound(got, want, "mha decode")


def test_mha_decode_batched_with_per_sequence_lengths_on_device(K):
    import torch

    rng = np.random.default_rng(9)
    B, H, G, D, S = 5, 32, 8, 64, 256
    q = normal(rng, (B, H, D))
    k, v = normal(rng, (B, S, G, D)), normal(rng, (B, S, G, D))
    pos = np.array([0, 17, 100, 254, 63], np.int32)   # kv_valid = position + 1
    ns = 4
    got = to_numpy(K.mha_decode(to_torch(q), to_torch(k), to_torch(v), d_kv_valid=to_torch(pos),
                                per_batch=True, kv_valid_add=1, nsplit=ns))
    for b in range(B):
        want = ops.mha(q[b : b + 1], k[b], v[b], num_heads=H, num_kv_heads=G, heads_interleaved=True,
                       kv_interleaved=True, q_tokens=1, kv_tokens=int(pos[b]) + 1)
        assert_verdict(got[b : b + 1], want, MHA_TOL, what=f"sequence {b}")


@pytest.mark.parametrize("B,H,G,D,S,window", [
    (40, 32, 8, 64, 300, None),     # 320 (sequence, KV head) pairs: the tensor-core kernel
    (64, 24, 8, 128, 200, None),    # 128-wide heads, groups of 3
    (300, 5, 1, 64, 130, 40),       # groups of 5, one KV head, a sliding window
    (38, 32, 8, 64, 129, None),
    (8, 24, 8, 128, 2304, None),    # 64 pairs do not fill the machine: the keys are split over clusters of four
    (8, 32, 8, 64, 1100, 300),      # clusters of four, a sliding window that leaves some splits empty
    (16, 8, 2, 128, 4608, None),    # clusters of eight
])
def test_mha_decode_large_batches_on_the_tensor_cores(K, B, H, G, D, S, window):
    """A batch that fills the machine takes the MMA kernel: every sequence has its own
    length (empty, one key, tile boundaries, full)."""
    rng = np.random.default_rng(12)
    q = normal(rng, (B, H, D))
    k, v = normal(rng, (B, S, G, D)), normal(rng, (B, S, G, D))
    pos = rng.integers(0, S, B).astype(np.int32)
    pos[:6] = [0, 63, 64, 127, 128, S - 1]
    got = to_numpy(K.mha_decode(to_torch(q), to_torch(k), to_torch(v), d_kv_valid=to_torch(pos),
                                per_batch=True, kv_valid_add=1, window=window))
    for b in list(range(8)) + [B // 2, B - 1]:
        want = ops.mha(q[b : b + 1], k[b], v[b], num_heads=H, num_kv_heads=G, window=window,
                       heads_interleaved=True, kv_interleaved=True, q_tokens=1, kv_tokens=int(pos[b]) + 1)
        assert_verdict(got[b : b + 1], want, MHA_TOL, what=f"sequence {b} of {B}")
        assert_bf16_bound(got[b : b + 1], want, f"sequence {b} of {B}")
    # a sequence with no keys at all gives zeros
    zero = to_numpy(K.mha_decode(to_torch(q), to_torch(k), to_torch(v), kv_valid=0))
    assert not zero.any()


def test_mha_decode_non_interleaved_cache_layout(K):
    rng = np.random.default_rng(10)
    H, G, D, S = 8, 2, 64, 512
    q = normal(rng, (1, H, D))
    k, v = normal(rng, (G, S, D)), normal(rng, (G, S, D))
    want = ops.mha(np.swapaxes(q, 0, 1), k, v, num_heads=H, num_kv_heads=G, q_tokens=1, kv_tokens=S)
    ns = 4
    got = to_numpy(K.mha_decode(to_torch(q), to_torch(k), to_torch(v), kv_valid=S, nsplit=ns, kv_interleaved=False))
    assert_verdict(got.reshape(H, 1, D), want, MHA_TOL)
