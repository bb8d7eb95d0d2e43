"""The encoder-side element-wise and row-wise kernels against their operators' references (B200).

The catalogue walk covers every default case; here the per-call bounds (rows of LayerNorm, the
column bound of Softmax at lengths that are not whole vectors, in immediate and device
form), error returns and the exact operators' bit-equality.
"""

import numpy as np
import pytest
from ml_dtypes import bfloat16

from iron_b200.operators import GELU, Clamp, LayerNorm, ReLU, Softmax, Tanh
from iron_b200.verify import Tolerance
from tests.util import assert_bf16_bound, assert_verdict, normal, to_numpy, to_torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def K():
    from iron_b200 import kernels

    return kernels


@pytest.mark.parametrize("n", [8, 2048, 65536 + 24, 1000003])
def test_unary_operators_follow_their_references_at_ragged_sizes(K, n):
    rng = np.random.default_rng(n)
    x = normal(rng, (n,), scale=3.0)
    for op, name in ((ReLU(size=n), "relu"), (Tanh(size=n), "tanh"), (GELU(size=n), "gelu_tanh"),
                     (GELU(size=n, approximate="none"), "gelu_erf")):
        got = to_numpy(K.elementwise(name, to_torch(x)))
        want = op.reference(x)
        assert_verdict(got, want, Tolerance.bf16_ulps(1, atol=1e-6), what=f"{name} n={n}")
        assert_bf16_bound(got, want, what=name)
    relu = to_numpy(K.elementwise("relu", to_torch(x)))
    assert np.array_equal(relu.view(np.uint16), ReLU(size=n).reference(x).view(np.uint16))


@pytest.mark.parametrize("low,high", [(-0.75, 1.25), (0.5, 1.5), (-3e4, 3e4), (0.3, 0.3)])
def test_clamp_is_exact_and_rounds_its_bounds_to_bf16(K, low, high):
    rng = np.random.default_rng(7)
    x = normal(rng, (4099,), scale=2.0)
    got = to_numpy(K.clamp(to_torch(x), low, high))
    want = Clamp(size=4099, low=low, high=high).reference(x)
    assert np.array_equal(got.view(np.uint16), want.view(np.uint16))
    from iron_b200._lib import IronError

    with pytest.raises(IronError):
        K.clamp(to_torch(x), 1.0, -1.0)


@pytest.mark.parametrize("rows,cols,weighted", [(1, 2048, True), (32, 512, False), (197, 768, True), (64, 8, True)])
def test_layer_norm_rows_and_bounds(K, rows, cols, weighted):
    import torch

    rng = np.random.default_rng(rows)
    x = (normal(rng, (rows, cols), scale=2.0).astype(np.float32) + 0.5).astype(bfloat16)
    w = (1 + normal(rng, (cols,), scale=0.1).astype(np.float32)).astype(bfloat16) if weighted else None
    op = LayerNorm(rows=rows, tile_size=cols, weighted=weighted, epsilon=1e-5)
    want = op.reference(x, w) if weighted else op.reference(x)
    got = to_numpy(K.layer_norm(to_torch(x), to_torch(w) if weighted else None, eps=1e-5))
    assert_verdict(got, want, op.tolerance(), what=f"LayerNorm {rows}x{cols}")
    assert_bf16_bound(got, want, what="LayerNorm")
    if rows > 1:
        out = torch.full((rows, cols), 7.0, dtype=torch.bfloat16, device="cuda")
        valid = rows // 2
        K.layer_norm(to_torch(x), to_torch(w) if weighted else None, out, eps=1e-5, valid=valid)
        o = to_numpy(out)
        assert np.array_equal(o[:valid].view(np.uint16), got[:valid].view(np.uint16))
        assert (o[valid:].astype(np.float32) == 7.0).all()
        d = torch.tensor([valid], dtype=torch.int32, device="cuda")
        out.fill_(7.0)
        K.layer_norm(to_torch(x), to_torch(w) if weighted else None, out, eps=1e-5, d_valid=d)
        assert np.array_equal(to_numpy(out).view(np.uint16), o.view(np.uint16))


@pytest.mark.parametrize("rows,cols,length", [(32, 1024, None), (16, 4608, 4001), (16, 512, 1), (16, 64, 0),
                                             (32, 32768, 32768), (16, 2048, 1027)])
def test_softmax_over_a_bounded_run_of_columns(K, rows, cols, length):
    import torch

    rng = np.random.default_rng(cols)
    x = normal(rng, (rows, cols), scale=3.0)
    op = Softmax(rows=rows, cols=cols)
    op = op if length is None else op.bind(length=length)
    want = op.reference(x)
    got = to_numpy(K.softmax(to_torch(x), length=length))
    assert_verdict(got, want, op.tolerance(), what=f"Softmax {rows}x{cols} n={length}")
    n = cols if length is None else length
    assert not got[:, n:].astype(np.float32).any()
    if n:
        assert np.abs(got.astype(np.float32).sum(-1) - 1).max() <= 2e-2
    if length is not None:
        d = torch.tensor([length], dtype=torch.int32, device="cuda")
        again = to_numpy(K.softmax(to_torch(x), d_length=d))
        assert np.array_equal(again.view(np.uint16), got.view(np.uint16))


@pytest.mark.parametrize("cap,addend", [(None, False), (50.0, True), (2.0, False), (None, True)])
def test_softmax_float32_input_with_soft_cap_and_addend(K, cap, addend):
    rng = np.random.default_rng(3)
    rows, cols = 64, 1504
    x = (rng.standard_normal((rows, cols)) * 6).astype(np.float32)
    a = (rng.standard_normal((rows, cols)) * 2).astype(np.float32) if addend else None
    op = Softmax(rows=rows, cols=cols, input_dtype=np.float32, soft_cap=cap, has_addend=addend)
    want = op.reference(x, a) if addend else op.reference(x)
    got = to_numpy(K.softmax(to_torch(x), addend=to_torch(a) if addend else None, soft_cap=cap))
    assert_verdict(got, want, op.tolerance(), what=f"Softmax f32 cap={cap} addend={addend}")
