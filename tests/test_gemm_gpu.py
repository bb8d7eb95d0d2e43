"""The tcgen05 GEMM against the oracle's GEMM / ProjectionGEMM references (B200).

Tolerance is the reference's own bound, ``2 * 2^-8 * |A| @ |B|`` elementwise
(iron/operators/gemm.py:704-735, HIGHEST precision), plus the bf16 output bound (1e-2 relative / 2e-2 absolute).
"""

import numpy as np
import pytest
from ml_dtypes import bfloat16

from iron_b200.verify import Tolerance, compare
from oracle import ops
from tests.util import assert_bf16_bound, normal, to_numpy, to_torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def K():
    from iron_b200 import kernels

    return kernels


def check(got, A, B, want, b_col_maj=False, c_col_maj=False, what=""):
    bound = ops.gemm_bound(A, B, b_col_maj=b_col_maj, c_col_maj=c_col_maj)
    v = compare(got, want, Tolerance.bounded(lambda *a: bound), bound=bound)
    assert v, f"{what}: {v.detail}"


CASES = [
    # M, N, K -- the reference's GEMM cases are multiples of 64; ragged ones added
    (128, 64, 64), (128, 256, 64), (256, 256, 256), (2048, 2048, 2048), (2048, 512, 2048),
    (384, 1536, 768), (200, 96, 136), (130, 520, 72), (64, 8192, 2048), (2048, 2048, 8192),
    (2048, 3072, 512), (1500, 3000, 264),   # CTA pairs with 192-column tiles (fewer waves than 256), ragged too
]


@pytest.mark.parametrize("M,N,Kd", CASES)
@pytest.mark.parametrize("b_col_maj", [True, False])
def test_gemm_matches_reference(K, M, N, Kd, b_col_maj):
    rng = np.random.default_rng(1001)
    A = normal(rng, (M, Kd), 1 / np.sqrt(Kd))
    B = normal(rng, (N, Kd) if b_col_maj else (Kd, N), 1.0)
    if not b_col_maj and N % 8:
        pytest.skip("row pitch of B must be a multiple of 8")
    want = ops.gemm(A, B, b_col_maj=b_col_maj)
    got = to_numpy(K.gemm(to_torch(A), to_torch(B), b_col_maj=b_col_maj))
    check(got, A, B, want, b_col_maj, what=f"{M}x{N}x{Kd} b_col_maj={b_col_maj}")


SKINNY = [
    # rows, N, K: a decode batch against weights as stored -- the weight-streaming kernel with the
    # operands swapped: split along K over clusters of 8, 4, 2 CTAs, one CTA a tile, ragged edges
    (64, 2048, 2048), (64, 2048, 8192), (33, 3072, 2048), (5, 4096, 1024), (1, 2048, 2048),
    (64, 8192, 2048), (17, 200, 136), (64, 18944, 512), (8, 1000, 72),
]


@pytest.mark.parametrize("rows,N,Kd", SKINNY)
@pytest.mark.parametrize("residual", [False, True], ids=["plain", "residual"])
def test_a_decode_batch_streams_the_weights(K, rows, N, Kd, residual):
    import torch

    rng = np.random.default_rng(rows + N + Kd)
    A = normal(rng, (rows, Kd), 1 / np.sqrt(Kd))
    W = normal(rng, (N, Kd), 1.0)
    res = normal(rng, (rows, N), 1.0) if residual else None
    want = ops.gemm(A, W, b_col_maj=True)
    if residual:
        want = ops.add(want, res)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    got = to_numpy(K.gemm(to_torch(A), to_torch(W), b_col_maj=True, residual=to_torch(res) if residual else None,
                          status=status))
    bound = ops.gemm_bound(A, W, b_col_maj=True) + (np.abs(res.astype(np.float32)) * 2 ** -8 if residual else 0)
    v = compare(got, want, Tolerance.bounded(lambda *a: bound), bound=bound)
    assert v, f"{rows}x{N}x{Kd}: {v.detail}"
    assert int(status.item()) == 0


def test_gemm_2048_cubed_within_the_bf16_output_bound(K):
    rng = np.random.default_rng(1001)
    A = normal(rng, (2048, 2048), 1 / np.sqrt(2048))
    B = normal(np.random.default_rng(1002), (2048, 2048), 1 / np.sqrt(2048))
    for b_col_maj in (False, True):
        want = ops.gemm(A, B, b_col_maj=b_col_maj)
        got = to_numpy(K.gemm(to_torch(A), to_torch(B), b_col_maj=b_col_maj))
        assert_bf16_bound(got, want, f"b_col_maj={b_col_maj}")


def test_bounded_rows_are_neither_computed_nor_written(K):
    import torch

    rng = np.random.default_rng(3)
    A, B = normal(rng, (512, 256), 1 / 16), normal(rng, (384, 256))
    out = torch.full((512, 384), 5.0, dtype=torch.bfloat16, device="cuda")
    nv = torch.tensor([300], dtype=torch.int32, device="cuda")
    K.gemm(to_torch(A), to_torch(B), out, b_col_maj=True, d_valid=nv)
    got = to_numpy(out)
    check(got[:300], A[:300], B, ops.gemm(A[:300], B, b_col_maj=True), True)
    assert (got[300:].astype(np.float32) == 5.0).all()


def test_bounded_k(K):
    rng = np.random.default_rng(4)
    A, B = normal(rng, (256, 512), 1 / 16), normal(rng, (512, 256))
    got = to_numpy(K.gemm(to_torch(A), to_torch(B), valid_k=200))
    check(got, A[:, :200], B[:200], ops.gemm(A, B, valid_k=200))


@pytest.mark.parametrize("epilogue", ["silu", "sigmoid"])
def test_projection_gemm_output_stage(K, epilogue):
    rng = np.random.default_rng(5)
    A, W = normal(rng, (256, 512), 1 / 16), normal(rng, (768, 512))
    want = ops.projection_gemm(A, W, epilogue=epilogue)
    got = to_numpy(K.gemm(to_torch(A), to_torch(W), b_col_maj=True, epilogue=epilogue))
    # The reference states no tolerance for an activated GEMM (flm/gemm/op.py:1355-1356):
    # a one-ulp difference of the rounded product is amplified by the activation's own
    # two roundings.
    v = compare(got, want, Tolerance.relative(0.02, atol=2e-2))
    assert v, v.detail


def test_residual_and_transposed_and_f32_outputs(K):
    rng = np.random.default_rng(6)
    A, W = normal(rng, (300, 256), 1 / 16), normal(rng, (520, 256))
    res = normal(rng, (300, 520))
    want = ops.add(res, ops.gemm(A, W, b_col_maj=True))
    got = to_numpy(K.gemm(to_torch(A), to_torch(W), b_col_maj=True, residual=to_torch(res)))
    v = compare(got, want, Tolerance.bf16_ulps(2, atol=2e-2))
    assert v, v.detail
    wantT = ops.gemm(A, W, b_col_maj=True, c_col_maj=True)
    gotT = to_numpy(K.gemm(to_torch(A), to_torch(W), b_col_maj=True, c_col_maj=True))
    check(gotT, A, W, wantT, True, True)
    want32 = ops.gemm(A, W, b_col_maj=True, output_dtype=np.float32)
    got32 = to_numpy(K.gemm(to_torch(A), to_torch(W), b_col_maj=True, out_f32=True))
    assert np.allclose(got32, want32, rtol=1e-4, atol=1e-4)


def test_no_pipeline_wait_gave_up(K):
    import torch

    rng = np.random.default_rng(7)
    A, W = normal(rng, (1024, 1024), 1 / 32), normal(rng, (1024, 1024))
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    K.gemm(to_torch(A), to_torch(W), b_col_maj=True, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0


@pytest.mark.parametrize("M,N,Kd", [(128, 128, 64), (2048, 8192, 2048), (64, 8192, 2048), (200, 328, 136), (7, 2048, 512), (5, 328, 136), (33, 5000, 320)])
def test_gated_two_weight_form_matches_the_chain_of_references(K, M, N, Kd):
    """gate GEMM, up GEMM, SiLU, product -- each rounded as the separate operators round."""
    rng = np.random.default_rng(1010)
    A = normal(rng, (M, Kd), 1.0)
    Wg = normal(rng, (N, Kd), 1 / np.sqrt(Kd))
    Wu = normal(rng, (N, Kd), 1 / np.sqrt(Kd))
    gate, up = ops.gemm(A, Wg, b_col_maj=True), ops.gemm(A, Wu, b_col_maj=True)
    want = ops.mul(ops.silu(gate), up)
    got = to_numpy(K.gemm_swiglu(to_torch(A), to_torch(Wg), to_torch(Wu)))
    assert got.shape == (M, N)
    # A one-ulp flip of gate or of up (f32 sums in another order) moves the product by one
    # of its own ulps, 2^-8 relative: all but a few in a million elements are inside the
    # bf16 output bound (1e-2 relative / 2e-2 absolute), and none is further than two ulps.
    err = np.abs(got.astype(np.float64) - want.astype(np.float64))
    scale = np.abs(want.astype(np.float64))
    inside = (err <= 1e-2 * scale) | (err <= 2e-2)
    assert inside.mean() >= 1 - 1e-5, f"{M}x{N}x{Kd}: {int((~inside).sum())} of {inside.size} outside the bound"
    assert (err <= 2 ** -6 * scale + 2e-2).all()
    # and it is what the three separate launches give: bit for bit where both walk K in the
    # same order, a rounding flip here and there where the skinny separate GEMMs split K
    g = K.gemm(to_torch(A), to_torch(Wg), b_col_maj=True)
    u = K.gemm(to_torch(A), to_torch(Wu), b_col_maj=True)
    chain = to_numpy(K.elementwise("silu_mul", g, u))
    same = got.view(np.uint16) == chain.view(np.uint16)
    if M >= 128:
        assert same.all()
    else:
        d = np.abs(got.astype(np.float64) - chain.astype(np.float64))
        assert same.mean() >= 0.99 and (d <= 2 ** -6 * np.abs(chain.astype(np.float64)) + 2e-2).all()


@pytest.mark.parametrize("rows,H,G,D,Kd,start", [(512, 16, 4, 64, 512, 0), (300, 8, 2, 64, 264, 37),
                                                 (256, 6, 2, 128, 256, 5), (2048, 32, 8, 64, 2048, 0)])
def test_the_fused_qkv_projection_equals_the_projection_then_the_rope_kernel_bit_for_bit(K, rows, H, G, D, Kd, start):
    import torch

    from oracle.model import rope_angles

    rng = np.random.default_rng(rows + D)
    S = start + rows + 3
    x = to_torch(normal(rng, (rows, Kd), 1.0))
    w = to_torch(normal(rng, ((H + 2 * G) * D, Kd), 1 / np.sqrt(Kd)))
    angles = to_torch(rope_angles(D, S, 500000.0).astype(np.float32)).to(torch.bfloat16)
    N = (H + 2 * G) * D

    def caches():
        return (torch.full((S, G, D), 3.0, dtype=torch.bfloat16, device="cuda"),
                torch.full((S, G, D), 3.0, dtype=torch.bfloat16, device="cuda"))

    k0, v0 = caches()
    qkv0 = torch.empty(rows, N, dtype=torch.bfloat16, device="cuda")
    K.gemm(x, w, qkv0, b_col_maj=True)
    K.rope_kv_write(qkv0, angles, k0, v0, rows=rows, H=H, G=G, D=D, start=start)
    k1, v1 = caches()
    qkv1 = torch.zeros(rows, N, dtype=torch.bfloat16, device="cuda")
    assert K.gemm_qkv_rope(x, w, qkv1, angles, k1, v1, H=H, G=G, D=D, start=start)
    bits = lambda t: to_numpy(t).view(np.uint16)
    assert np.array_equal(bits(qkv1[:, : H * D]), bits(qkv0[:, : H * D]))       # the rotated queries
    assert np.array_equal(bits(k1), bits(k0)) and np.array_equal(bits(v1), bits(v0))   # rows outside stay 3.0
    # one row tile is not the pair GEMM's: nothing is launched and the caller is told
    assert not K.gemm_qkv_rope(x[:64], w, qkv1[:64], angles, k1, v1, H=H, G=G, D=D, start=start)


def test_residual_rows_off_the_16_byte_grid_take_the_scalar_path(K):
    """N = 100: rows of the output and of the residual start every 200 bytes, so neither the
    residual read nor the store may be a 16-byte access; the result is the chain's."""
    rng = np.random.default_rng(1020)
    A, W = normal(rng, (256, 64), 1 / 8), normal(rng, (100, 64))
    res = normal(rng, (256, 100))
    want = ops.add(ops.gemm(A, W, b_col_maj=True), res)
    got = to_numpy(K.gemm(to_torch(A), to_torch(W), b_col_maj=True, residual=to_torch(res)))
    v = compare(got, want, Tolerance.bf16_ulps(2, atol=2e-2))
    assert v, v.detail
