"""The projections of a batched decode step with their neighbours folded in, on a B200.

``gemm_rows`` / ``gemm_rows_qkv_rope`` are the weight-streaming GEMM of a decode batch with
the RMSNorm before it and the RoPE + cache write after it inside the launch
(iron/lm/blocks.py chains them as separate operators).  Each is checked against the separate
kernels it replaces -- the same bits where the arithmetic is the same operations in the same
order (RoPE, the residual), two bf16 ulps where only the order of a float32 sum of squares
differs (the folded norm) -- and the sums of squares against the oracle.
"""

import numpy as np
import pytest
from ml_dtypes import bfloat16

from iron_b200.verify import Tolerance
from oracle import ops
from tests.util import assert_verdict, normal, to_numpy, to_torch

pytestmark = pytest.mark.gpu

# The folded norm adds the squares in another order than the norm kernel: 1/rms may differ in its last
# float32 bit, a normalised value in a row may then round to the neighbouring bf16, and an output of
# that row moves by that one term (about 3e-4 here) -- two ulps, or that much near zero.
NEAR = Tolerance.bf16_ulps(2, atol=2e-3)
# ... and through silu(gate) * up a gate that moved by one ulp moves the product by up to that ulp times up
GATED = Tolerance.relative(rtol=0.01, atol=2e-3)


@pytest.fixture(scope="module")
def K():
    from iron_b200 import kernels

    return kernels


# rows, H, G, D, hidden: Llama-3.2-1B and 3B head shapes, a ragged batch, a small case whose K is not split
QKV = [(64, 32, 8, 64, 2048), (5, 32, 8, 64, 2048), (64, 24, 8, 128, 3072), (33, 2, 2, 64, 512), (7, 2, 1, 128, 256)]


@pytest.mark.parametrize("rows,H,G,D,E", QKV)
def test_qkv_with_rope_and_cache_write_matches_the_separate_kernels(K, rows, H, G, D, E):
    import torch

    rng = np.random.default_rng(rows + H + D + E)
    S = 40
    x = to_torch(normal(rng, (rows, E), 1.0))
    w = to_torch(normal(rng, ((H + 2 * G) * D, E), 1 / np.sqrt(E)))
    angles = to_torch(normal(rng, (S, D)))
    positions = torch.tensor(rng.integers(0, S, rows), dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")

    def caches():
        return (torch.full((rows, S, G, D), 3.0, dtype=torch.bfloat16, device="cuda"),
                torch.full((rows, S, G, D), 4.0, dtype=torch.bfloat16, device="cuda"))

    want_k, want_v = caches()
    want_q = torch.empty(rows, H, D, dtype=torch.bfloat16, device="cuda")
    qkv = K.gemm(x, w, b_col_maj=True, status=status)
    K.rope_kv_scatter(qkv, angles, want_q, want_k, want_v, positions, H=H, G=G, D=D)

    got_k, got_v = caches()
    got_q = torch.empty_like(want_q)
    K.gemm_rows_qkv_rope(x, w, angles, got_q, got_k, got_v, positions, H=H, G=G, D=D, status=status)
    assert torch.equal(got_q, want_q)
    assert torch.equal(got_k, want_k) and torch.equal(got_v, want_v)   # the other cache rows untouched too
    assert int(status.item()) == 0


# rows, hidden, inner (o_proj-like K), F: one layer's chain; Llama-1B, 3B-like, small and ragged
CHAIN = [(64, 2048, 2048, 8192), (9, 2048, 2048, 8192), (64, 3072, 3072, 8192), (21, 512, 256, 1024), (3, 200, 64, 136)]


@pytest.mark.parametrize("rows,E,inner,F", CHAIN)
def test_a_folded_norm_matches_the_norm_kernel_and_the_sums_match_the_oracle(K, rows, E, inner, F):
    import torch

    rng = np.random.default_rng(rows + E + F)
    att = to_torch(normal(rng, (rows, inner), 1.0))
    wo = to_torch(normal(rng, (E, inner), 1 / np.sqrt(inner)))
    x = to_torch(normal(rng, (rows, E), 1.0))
    ln = to_torch((1 + rng.standard_normal(E, dtype=np.float32) / 10).astype(bfloat16))
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    sums = K.rowsq_buffer()

    # the producer: o_proj + residual, leaving the rows' sums of squares
    y = K.gemm_rows(att, wo, residual=x, rowsq_out=sums, status=status)
    assert torch.equal(y, K.gemm(att, wo, b_col_maj=True, residual=x, status=status))
    parts = K.gemm_rows_parts(rows, E, inner)
    assert parts > 0
    got_sums = sums[:rows, :parts].double().sum(dim=1).cpu().numpy()
    want_sums = (to_numpy(y).astype(np.float64) ** 2).sum(axis=1)
    assert np.allclose(got_sums, want_sums, rtol=1e-5), np.abs(got_sums / want_sums - 1).max()
    if E % 64:
        return   # the folded norm wants whole k blocks: such a model keeps the norm kernel

    # consumers: the gated pair and a plain projection behind the folded norm
    wg = to_torch(normal(rng, (F, E), 1 / np.sqrt(E)))
    wu = to_torch(normal(rng, (F, E), 1 / np.sqrt(E)))
    h = K.rms_norm(y, ln, eps=1e-5)
    want = K.gemm_swiglu(h, wg, wu, status=status)
    got = K.gemm_rows(y, wg, W2=wu, norm_weight=ln, rowsq_in=sums, rowsq_parts=parts, eps=1e-5, status=status)
    assert_verdict(to_numpy(got), to_numpy(want), GATED, what="gate/up behind a folded norm")
    assert float((got != want).float().mean()) < 0.01
    want = K.gemm(h, wg, b_col_maj=True, status=status)
    got = K.gemm_rows(y, wg, norm_weight=ln, rowsq_in=sums, rowsq_parts=parts, eps=1e-5, status=status)
    assert_verdict(to_numpy(got), to_numpy(want), NEAR, what="projection behind a folded norm")
    assert float((got != want).float().mean()) < 0.01
    # and against the oracle's norm + product, within the product's own rounding bound
    hn = ops.rms_norm(to_numpy(y), to_numpy(ln), 1e-5)
    ref = ops.gemm(hn, to_numpy(wg), b_col_maj=True)
    bound = ops.gemm_bound(hn, to_numpy(wg), b_col_maj=True) * 2
    assert np.all(np.abs(to_numpy(got).astype(np.float32) - ref.astype(np.float32)) <= bound)
    assert int(status.item()) == 0


def test_qkv_with_norm_and_rope_folded_in(K):
    """All three at once, as a layer after the first calls it: down_proj's sums feed the norm."""
    import torch

    rows, E, F, H, G, D, S = 64, 2048, 8192, 32, 8, 64, 24
    rng = np.random.default_rng(11)
    act = to_torch(normal(rng, (rows, F), 1.0))
    wd = to_torch(normal(rng, (E, F), 1 / np.sqrt(F)))
    y = to_torch(normal(rng, (rows, E), 1.0))
    ln = to_torch((1 + rng.standard_normal(E, dtype=np.float32) / 10).astype(bfloat16))
    w = to_torch(normal(rng, ((H + 2 * G) * D, E), 1 / np.sqrt(E)))
    angles = to_torch(normal(rng, (S, D)))
    positions = torch.tensor(rng.integers(0, S, rows), dtype=torch.int32, device="cuda")
    sums = K.rowsq_buffer()
    x = K.gemm_rows(act, wd, residual=y, rowsq_out=sums)
    parts = K.gemm_rows_parts(rows, E, F)

    want_k = torch.zeros(rows, S, G, D, dtype=torch.bfloat16, device="cuda")
    want_v, got_k, got_v = torch.zeros_like(want_k), torch.zeros_like(want_k), torch.zeros_like(want_k)
    want_q = torch.empty(rows, H, D, dtype=torch.bfloat16, device="cuda")
    got_q = torch.empty_like(want_q)
    K.rope_kv_scatter(K.gemm(K.rms_norm(x, ln, eps=1e-5), w, b_col_maj=True), angles, want_q, want_k, want_v,
                      positions, H=H, G=G, D=D)
    K.gemm_rows_qkv_rope(x, w, angles, got_q, got_k, got_v, positions, H=H, G=G, D=D, norm_weight=ln,
                         rowsq_in=sums, rowsq_parts=parts, eps=1e-5)
    for got, want, what in ((got_q, want_q, "q"), (got_k, want_k, "k cache"), (got_v, want_v, "v cache")):
        assert_verdict(to_numpy(got), to_numpy(want), NEAR, what=what)
        assert float((got != want).float().mean()) < 0.01


def test_what_the_folded_forms_refuse(K):
    import torch

    from iron_b200._lib import IronError

    x = torch.zeros(4, 256, dtype=torch.bfloat16, device="cuda")
    w = torch.zeros(128, 256, dtype=torch.bfloat16, device="cuda")
    ln = torch.ones(256, dtype=torch.bfloat16, device="cuda")
    sums = K.rowsq_buffer()
    with pytest.raises(ValueError):                      # a norm without its sums
        K.gemm_rows(x, w, norm_weight=ln)
    with pytest.raises(IronError):                       # sums of squares only of a residual stream
        K.gemm_rows(x, w, rowsq_out=sums)
    with pytest.raises(IronError):                       # no slots
        K.gemm_rows(x, w, norm_weight=ln, rowsq_in=sums, rowsq_parts=0)
    with pytest.raises(IronError):                       # more than 64 rows is the general GEMM's
        K.gemm_rows(torch.zeros(65, 256, dtype=torch.bfloat16, device="cuda"), w)
    with pytest.raises(IronError):                       # a head width the 128-row tile does not hold whole
        K.gemm_rows_qkv_rope(x, torch.zeros(4 * 32, 256, dtype=torch.bfloat16, device="cuda"),
                             torch.zeros(8, 32, dtype=torch.bfloat16, device="cuda"),
                             torch.zeros(4, 2, 32, dtype=torch.bfloat16, device="cuda"),
                             torch.zeros(4, 8, 1, 32, dtype=torch.bfloat16, device="cuda"),
                             torch.zeros(4, 8, 1, 32, dtype=torch.bfloat16, device="cuda"),
                             torch.zeros(4, dtype=torch.int32, device="cuda"), H=2, G=1, D=32)
