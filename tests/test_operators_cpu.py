"""Operator classes without a device: declaration, construction errors, inference, judging.

What iron/tests/common/test_declare.py and iron/tests/common/test_judging.py:74-110 pin in the
reference: keyword-only construction, shapes from fields, fields from shapes, ``step`` outside
a body, and that every operator's own reference passes its own tolerance while a NaN or a
value well past the tolerance fails.
"""

import numpy as np
import pytest
from ml_dtypes import bfloat16

from iron_b200.operators import CATALOG, GEMM, GEMV, MHA, RMSNorm, RoPE, SelectiveScan
from iron_b200.testing import vectors
from iron_b200.verify import Tolerance, compare
from oracle import ops as oracle


def small_case(cls):
    cases = [c for c in cls.test.resolve(cls) if not c.extensive]
    sized = sorted(cases, key=lambda c: np.prod([v for v in c.kwargs.values() if isinstance(v, int)], dtype=float))
    return sized[0]


@pytest.mark.parametrize("cls", CATALOG, ids=lambda c: c.__name__)
def test_the_reference_passes_its_own_tolerance_and_faults_do_not(cls):
    case = small_case(cls)
    if cls is MHA:
        case = type(case)(dict(num_heads=4, num_KV_heads=2, seq_len=64, kv_len=128))
    if cls.__name__ in ("GEMM", "ProjectionGEMM"):
        case = type(case)(dict(case.kwargs, M=64, K=64, N=64))
    op = cls(**case.kwargs)
    extra = cls.test.draw(op) if cls.test.draw else {}
    vec = vectors(op, seed=42, **extra)
    tol = op.tolerance()
    if tol is None:
        pytest.skip("the operator states no tolerance")
    verdicts = op.judge(vec.inputs, vec.outputs, tol)
    assert all(verdicts.values()), {n: v.detail for n, v in verdicts.items()}
    name = next(n for n, a in vec.outputs.items() if a.dtype.kind == "f" or a.dtype == bfloat16) \
        if any(a.dtype.kind == "f" or a.dtype == bfloat16 for a in vec.outputs.values()) else None
    if name is not None:
        broken = {n: np.array(a) for n, a in vec.outputs.items()}
        flat = broken[name].reshape(-1)
        flat[: max(1, flat.size // 50)] = np.nan
        assert not op.judge(vec.inputs, broken, tol, expected=vec.outputs)[name]


def test_construction_is_keyword_only_and_refuses_what_it_cannot_run():
    with pytest.raises(TypeError):
        GEMV(128, 64)
    with pytest.raises(TypeError):
        GEMV(M=128)
    with pytest.raises(TypeError):
        GEMV(M=128, K=64, columns=3)
    with pytest.raises(ValueError):
        GEMV(M=128, K=60)
    with pytest.raises(ValueError):
        RoPE(rows=8, cols=48)
    with pytest.raises(ValueError):
        RoPE(rows=8, cols=64, angle_rows=3)
    with pytest.raises(ValueError):
        SelectiveScan(rows=4, heads=3, head_dim=16, state_size=16, groups=2)
    with pytest.raises(TypeError):
        GEMV.step(np.zeros((8, 8)), np.zeros(8))
    # AIE tunables are accepted and carried, not used
    op = GEMV(M=128, K=64, num_aie_columns=8, tile_size_output=32)
    assert op.pinned == {"num_aie_columns", "tile_size_output"} and op.tile_size_output == 32


def test_shapes_follow_fields_and_fields_follow_shapes():
    g = GEMV(M=2048, K=64, num_batches=32, repeat=4)
    assert g.A.shape == (8, 2048, 64) and g.B.shape == (32, 64) and g.C.shape == (32, 2048)
    assert GEMV.declaration.infer({"A": (2048, 64), "B": (64,)}) == {"M": 2048, "K": 64, "num_batches": None}
    m = GEMM(M=4, K=8, N=16, b_col_maj=True, c_col_maj=True)
    assert m.B.shape == (16, 8) and m.C.shape == (16, 4)
    assert GEMM.declaration.infer({"A": (4, 8), "B": (16, 8)}, b_col_maj=True)["N"] == 16
    r = RMSNorm.declaration.infer({"x": (2, 64), "weight": (64,)})
    assert r == {"rows": 2, "tile_size": 64, "weighted": True}
    with pytest.raises(ValueError):
        GEMV.declaration.infer({"A": (128, 64), "B": (32,)})
    a = MHA(num_heads=32, num_KV_heads=8, seq_len=1, kv_len=2048, heads_interleaved=True)
    assert a.packed and a.seq_pad == 1 and a.Q.shape == (1, 32, 64) and a.K.shape == (8, 2048, 64)
    assert MHA(num_heads=8, seq_len=100).seq_pad == 128


def test_a_per_call_extent_reads_as_its_field_until_bound():
    g = GEMV(M=256, K=64)
    assert g.valid == 256 and g.bind(valid=100).valid == 100
    with pytest.raises(IndexError):
        g.bind(valid=257)
    with pytest.raises(TypeError):
        g.bind(rows=3)
    a = MHA(num_heads=4, num_KV_heads=2, seq_len=64, kv_len=256)
    assert a.q_tokens == 64 and a.kv_tokens == 256
    b = a.bind(valid=10, kv_valid=50)
    assert b.q_tokens == 10 and b.kv_tokens == 50


def test_operator_references_agree_with_the_oracle():
    rng = np.random.default_rng(0)
    A = rng.standard_normal((64, 32)).astype(bfloat16)
    x = rng.standard_normal(32).astype(bfloat16)
    assert np.array_equal(GEMV(M=64, K=32).reference(A, x), oracle.gemv(A, x))
    w = rng.standard_normal(32).astype(bfloat16)
    rows = rng.standard_normal((4, 32)).astype(bfloat16)
    assert np.array_equal(RMSNorm(rows=4, tile_size=32, weighted=True).reference(rows, w), oracle.rms_norm(rows, w))
    q = rng.standard_normal((64, 4, 64)).astype(bfloat16)
    k = rng.standard_normal((128, 2, 64)).astype(bfloat16)
    v = rng.standard_normal((128, 2, 64)).astype(bfloat16)
    op = MHA(num_heads=4, num_KV_heads=2, seq_len=64, kv_len=128, heads_interleaved=True, kv_interleaved=True)
    assert np.array_equal(op.reference(q, k, v), oracle.mha(q, k, v, num_heads=4, num_kv_heads=2,
                                                             heads_interleaved=True, kv_interleaved=True))
    bounded = op.bind(valid=10, kv_valid=40).reference(q, k, v)
    assert np.array_equal(bounded, oracle.mha(q, k, v, num_heads=4, num_kv_heads=2, heads_interleaved=True,
                                              kv_interleaved=True, q_tokens=10, kv_tokens=40))
    assert not bounded[10:].astype(np.float32).any()


def test_tolerance_edges():
    """iron/tests/common/test_judging.py:138-174: strict relative and atol, inclusive bound and range."""
    want = np.array([1.0, -2.0, 0.0, 100.0], np.float32)
    tol = Tolerance.relative(0.04, 1e-3)
    assert compare(want * 1.07, want, tol)                      # |a-b| < 0.04 (|a|+|b|)
    assert not compare(want * 1.10, want, tol)
    assert compare(want + 5e-4, want, tol).n_mismatch == 0
    assert compare(np.array([0.0009]), np.array([0.0]), tol) and not compare(np.array([0.001]), np.array([0.0]), tol)
    bounded = Tolerance.bounded(lambda x: 0.5 * np.ones_like(x))
    assert compare(want + 0.5, want, bounded, bound=0.5 * np.ones(4))
    assert not compare(want + 0.51, want, bounded, bound=0.5 * np.ones(4))
    assert compare(np.array([1.0, np.nan]), np.array([1.0, np.nan]), Tolerance.exact())
    assert not compare(np.array([1.0, np.nan]), np.array([1.0, 2.0]), tol)
    loose = Tolerance(rtol=0.0, atol=0.0, max_mismatch_frac=0.25)
    assert compare(np.array([1.0, 2.0, 3.0, 9.0]), np.array([1.0, 2.0, 3.0, 4.0]), loose)
    ulps = Tolerance.bf16_ulps(1)
    one = np.array([1.0], np.float32)
    assert compare(one + 2 ** -7, one, ulps) and not compare(one + 2 ** -6, one, ulps)


def test_host_refusals_come_before_any_launch():
    """What the kernels cannot run is refused on the host: a residual that is not laid out as
    the GEMM's output, and a decoder shape the fused engine has no kernels for."""
    import dataclasses

    import torch

    from iron_b200 import kernels as K
    from iron_b200.applications.llama.model import LlamaConfig
    from iron_b200.lm.engine import LlamaEngine

    A, W = torch.zeros(256, 64, dtype=torch.bfloat16), torch.zeros(100, 64, dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="residual"):
        K.gemm(A, W, b_col_maj=True, residual=torch.zeros(256, 104, dtype=torch.bfloat16)[:, :100])
    with pytest.raises(ValueError, match="residual"):
        K.gemm(A, W, b_col_maj=True, residual=torch.zeros(100, 256, dtype=torch.bfloat16))
    # the decode-batch projections with folded neighbours: a norm needs both its weight and the sums, sums and
    # residuals have fixed layouts, the q/k/v weight has (H + 2G) D rows
    X, ln = torch.zeros(4, 64, dtype=torch.bfloat16), torch.ones(64, dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="RMSNorm"):
        K.gemm_rows(X, W, norm_weight=ln)
    with pytest.raises(TypeError, match="rowsq"):
        K.gemm_rows(X, W, norm_weight=ln, rowsq_in=torch.zeros(64, 64), rowsq_parts=1)
    with pytest.raises(ValueError, match="residual"):
        K.gemm_rows(X, W, residual=torch.zeros(4, 104, dtype=torch.bfloat16)[:, :100])
    with pytest.raises(ValueError, match="do not chain"):
        K.gemm_rows(X, torch.zeros(100, 32, dtype=torch.bfloat16))
    with pytest.raises(ValueError, match="Wqkv"):
        K.gemm_rows_qkv_rope(X, W, ln, X, X, X, torch.zeros(4, dtype=torch.int32), H=1, G=1, D=64)
    base = LlamaConfig(vocab_size=64, hidden_size=64, num_hidden_layers=1, num_attention_heads=1,
                       num_key_value_heads=1, head_dim=64, intermediate_size=64, rope_theta=1e4, max_seq_len=8)
    for change in (dict(attention_bias=True), dict(mlp_bias=True), dict(hidden_act="gelu")):
        with pytest.raises(ValueError, match="LlamaEngine"):
            LlamaEngine(dataclasses.replace(base, **change), {})
