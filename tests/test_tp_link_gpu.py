"""A tensor-parallel exchange folded into the GEMVs on either side of it, on one B200.

The producing GEMV pushes its rows into every rank's exchange buffer, the consuming GEMV builds
its input from the ranks' slots plus the residual.  One GPU can play the whole protocol without
any kernel waiting on another: with a world of one the rank exchanges with itself, and with a
world of two both "ranks" are buffers on this GPU whose pushes are launched, in stream order,
before either pull -- every count a pull looks at is already there.  The last test lets a pull's
bounded wait run out (a second rank that never pushes): IRON_ERR_TIMEOUT in the status word,
nothing hangs, the context stays usable.
"""

import ctypes
import time

import numpy as np
import pytest
from ml_dtypes import bfloat16

from iron_b200.verify import Tolerance
from oracle import ops
from tests.util import assert_verdict, normal, to_numpy, to_torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def K():
    from iron_b200 import kernels

    return kernels


class Rank:
    """One rank's side of the exchange: its buffer, its eight state words, its status word."""

    def __init__(self, K, world, n):
        import torch

        self.buffer = torch.zeros(K.tp_buffer_bytes(world, n), dtype=torch.uint8, device="cuda")
        self.state = torch.zeros(8, dtype=torch.int32, device="cuda")
        self.status = torch.zeros(1, dtype=torch.int32, device="cuda")


def link(ranks, rank, n):
    peers = (ctypes.c_void_p * len(ranks))(*[r.buffer.data_ptr() for r in ranks])
    return dict(peer_buffers=peers, slot_elems=n, rank=rank, world=len(ranks), state=ranks[rank].state,
                status=ranks[rank].status)


def bf16_sum(parts, residual):
    """bf16(bf16(sum of the partials, in order, float32) + residual): what a pull builds."""
    acc = np.zeros(parts[0].shape, np.float32)
    for q in parts:
        acc = acc + q.astype(np.float32)
    return (acc.astype(bfloat16).astype(np.float32) + residual.astype(np.float32)).astype(bfloat16)


@pytest.mark.parametrize("E,inner,F", [(512, 256, 1024), (2048, 8192, 8192)],
                         ids=["small matrices", "large matrices (TMA-fed kernels)"])
def test_a_rank_exchanging_with_itself_reproduces_the_separate_steps(K, E, inner, F):
    """World of one, three exchanges in a row (both parities, the state advancing): o_proj-like
    push -> gate/up pull, down_proj-like push -> q/k/v pull, push -> head-like plain pull."""
    import torch

    rng = np.random.default_rng(E)
    me = [Rank(K, 1, E)]
    ln = (1 + rng.standard_normal(E, dtype=np.float32) / 10).astype(bfloat16)
    wo, att = normal(rng, (E, inner), 0.05), normal(rng, (inner,))
    wg, wu = normal(rng, (F, E), 0.05), normal(rng, (F, E), 0.05)
    wd = normal(rng, (E, F), 0.02)
    x = normal(rng, (E,))
    x_dev = to_torch(x)    # an attached exchange keeps raw addresses: the tensors outlive the launch that consumes it
    part = torch.empty(E, dtype=torch.bfloat16, device="cuda")
    unused = torch.zeros(E, dtype=torch.bfloat16, device="cuda")
    y = torch.empty(E, dtype=torch.bfloat16, device="cuda")

    # exchange 0: x + wo @ att -> y, consumed by the gated pair
    K.tp_push_next(**link(me, 0, E))
    K.gemv(to_torch(wo), to_torch(att), part)
    K.tp_pull_next(**link(me, 0, E), residual=x_dev, x_out=y)
    act = K.gemv_swiglu(to_torch(wg), to_torch(wu), unused, norm_weight=to_torch(ln), eps=1e-5)
    # the same kernel without an exchange adds the residual in its own last step: the same bits
    assert torch.equal(y, K.gemv(to_torch(wo), to_torch(att), residual=x_dev))
    want_y = to_numpy(y)
    assert_verdict(want_y, bf16_sum([ops.gemv(wo, att)], x), Tolerance.bf16_ulps(2), what="sum + residual")
    h = ops.rms_norm(want_y, ln, 1e-5)
    want_act = ops.mul(ops.silu(ops.gemv(wg, h)), ops.gemv(wu, h))
    assert_verdict(to_numpy(act), want_act, Tolerance.bf16_ulps(2), what="gate/up fed by an exchange")

    # exchange 1: y + wd @ act -> x2, consumed by a q/k/v projection with RoPE and the cache write
    H, G, D = 4, 2, 64
    wqkv = normal(rng, ((H + 2 * G) * D, E), 0.05)
    angles = to_torch(normal(rng, (8, D)))
    kc = torch.zeros(8, G, D, dtype=torch.bfloat16, device="cuda")
    vc = torch.zeros_like(kc)
    q = torch.empty(H, D, dtype=torch.bfloat16, device="cuda")
    x2 = torch.empty(E, dtype=torch.bfloat16, device="cuda")
    K.tp_push_next(**link(me, 0, E))
    K.gemv(to_torch(wd), act, part)
    K.tp_pull_next(**link(me, 0, E), residual=y, x_out=x2)
    K.decode_qkv_rope(to_torch(wqkv), unused, angles, kc, vc, q, H=H, G=G, D=D, position=3,
                      norm_weight=to_torch(ln), eps=1e-5)
    assert torch.equal(x2, K.gemv(to_torch(wd), act, residual=y))
    assert_verdict(to_numpy(x2), bf16_sum([ops.gemv(wd, to_numpy(act))], want_y), Tolerance.bf16_ulps(2),
                   what="second sum + residual")
    ref_q = torch.empty_like(q)
    ref_k, ref_v = torch.zeros_like(kc), torch.zeros_like(vc)
    K.decode_qkv_rope(to_torch(wqkv), x2, angles, ref_k, ref_v, ref_q, H=H, G=G, D=D, position=3,
                      norm_weight=to_torch(ln), eps=1e-5)
    assert torch.equal(q, ref_q) and torch.equal(kc, ref_k) and torch.equal(vc, ref_v)

    # exchange 2 (parity 0 again): a plain GEMV with a fused norm as the consumer, no residual
    head = normal(rng, (F, E), 0.05)
    K.tp_push_next(**link(me, 0, E))
    K.gemv(to_torch(wo), to_torch(att), part)
    K.tp_pull_next(**link(me, 0, E))
    logits = K.gemv(to_torch(head), unused, norm_weight=to_torch(ln), eps=1e-5)
    want = ops.gemv(head, ops.rms_norm(ops.gemv(wo, att), ln, 1e-5))
    assert_verdict(to_numpy(logits), want, Tolerance.bf16_ulps(2), what="plain GEMV fed by an exchange")
    torch.cuda.synchronize()
    assert me[0].state.tolist()[:2] == [3, 0] and int(me[0].status.item()) == 0


def test_two_ranks_on_one_gpu_sum_in_rank_order(K):
    """World of two, both ranks' buffers on this GPU: both pushes are launched before either pull."""
    import torch

    E, inner, F = 1024, 512, 2048
    rng = np.random.default_rng(2)
    ranks = [Rank(K, 2, E), Rank(K, 2, E)]
    w = [normal(rng, (E, inner), 0.05) for _ in range(2)]
    att = [normal(rng, (inner,)) for _ in range(2)]
    wg, wu = normal(rng, (F, E), 0.05), normal(rng, (F, E), 0.05)
    x = normal(rng, (E,))
    x_dev = to_torch(x)
    unused = torch.zeros(E, dtype=torch.bfloat16, device="cuda")
    part = torch.empty(E, dtype=torch.bfloat16, device="cuda")
    for round_ in range(2):   # both parities
        for r in range(2):
            K.tp_push_next(**link(ranks, r, E))
            K.gemv(to_torch(w[r]), to_torch(att[r]), part)
        want = bf16_sum([ops.gemv(w[0], att[0]), ops.gemv(w[1], att[1])], x)
        for r in range(2):
            y = torch.empty(E, dtype=torch.bfloat16, device="cuda")
            K.tp_pull_next(**link(ranks, r, E), residual=x_dev, x_out=y)
            act = K.gemv_swiglu(to_torch(wg), to_torch(wu), unused)
            assert np.array_equal(to_numpy(y).view(np.uint16), want.view(np.uint16)), (round_, r)
            want_act = ops.mul(ops.silu(ops.gemv(wg, want)), ops.gemv(wu, want))
            assert_verdict(to_numpy(act), want_act, Tolerance.bf16_ulps(2), what="two ranks' sum")
    assert all(int(r.status.item()) == 0 for r in ranks)
    assert ranks[0].state.tolist()[:2] == ranks[1].state.tolist()[:2] == [2, 0]


def test_what_the_exchange_refuses(K):
    import torch

    from iron_b200._lib import IronError

    E = 256
    me = [Rank(K, 1, E)]
    A = to_torch(normal(np.random.default_rng(0), (E, E)))
    v = torch.zeros(E, dtype=torch.bfloat16, device="cuda")
    K.tp_push_next(**link(me, 0, E))
    with pytest.raises(IronError):                      # a push takes no residual
        K.gemv(A, v, residual=v)
    assert K.gemv(A, v) is not None                     # the refused call consumed the link: this is a plain GEMV
    K.tp_push_next(**link(me, 0, E))
    with pytest.raises(IronError):                      # only the plain GEMV pushes
        K.gemv_swiglu(A, A, v)
    K.tp_pull_next(**link(me, 0, E // 2))
    with pytest.raises(IronError):                      # the vector does not fit a slot
        K.gemv(A, v)
    torch.cuda.synchronize()
    assert me[0].state.tolist() == [0] * 8


def test_a_rank_that_never_pushes_ends_the_pull_in_a_timeout_status(K):
    import torch

    E = 512
    ranks = [Rank(K, 2, E), Rank(K, 2, E)]
    A = to_torch(normal(np.random.default_rng(1), (E, E), 0.05))
    v = to_torch(normal(np.random.default_rng(2), (E,)))
    part = torch.empty(E, dtype=torch.bfloat16, device="cuda")
    K.tp_push_next(**link(ranks, 0, E))
    K.gemv(A, v, part)                                  # rank 0 pushes; rank 1 never does
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    K.tp_pull_next(**link(ranks, 0, E))
    out = K.gemv(A, v)
    torch.cuda.synchronize()
    waited = time.perf_counter() - t0
    assert int(ranks[0].status.item()) == -6            # IRON_ERR_TIMEOUT, reported not raised
    assert 1.0 < waited < 10.0
    assert ranks[0].state.tolist()[0] == 1              # the kernel ran to its end
    # it went on with what it had: rank 0's rows plus the absent rank's zeros
    want = ops.gemv(to_numpy(A), ops.gemv(to_numpy(A), to_numpy(v)))
    assert_verdict(to_numpy(out), want, Tolerance.bf16_ulps(2), what="after the timeout")
    # and the context is intact
    assert torch.equal(K.gemv(A, v), K.gemv(A, v))


@pytest.mark.parametrize("rows,E", [(1, 512), (8, 3072), (3, 200)], ids=["one row", "eight rows of 3072", "ragged"])
def test_the_all_reduce_over_tagged_words_with_one_rank_is_the_residual_add(K, rows, E):
    """World of one, four exchanges in a row (both parities twice, the state advancing): a batch's
    rows as one launch of many CTAs -- y = bf16(bf16(part) + residual)."""
    import torch

    rng = np.random.default_rng(rows * E)
    n = rows * E
    me = [Rank(K, 1, n)]
    for round_ in range(4):
        part, res = normal(rng, (rows, E)), normal(rng, (rows, E))
        y = torch.empty(rows, E, dtype=torch.bfloat16, device="cuda")
        K.tp_allreduce_tagged(to_torch(part), y, residual=to_torch(res), **link(me, 0, n))
        want = (part.astype(np.float32) + res.astype(np.float32)).astype(bfloat16)
        assert np.array_equal(to_numpy(y).view(np.uint16), want.view(np.uint16)), round_
        assert me[0].state.tolist()[:2] == [round_ + 1, 0]
    # without a residual: the partial itself
    part = normal(rng, (rows, E))
    y = torch.empty(rows, E, dtype=torch.bfloat16, device="cuda")
    K.tp_allreduce_tagged(to_torch(part), y, **link(me, 0, n))
    assert np.array_equal(to_numpy(y).view(np.uint16), part.view(np.uint16))
    assert int(me[0].status.item()) == 0


def test_the_all_reduce_over_tagged_words_gives_up_on_an_absent_rank(K):
    import torch

    n = 4 * 512
    ranks = [Rank(K, 2, n), Rank(K, 2, n)]
    rng = np.random.default_rng(5)
    part, res = normal(rng, (4, 512)), normal(rng, (4, 512))
    y = torch.empty(4, 512, dtype=torch.bfloat16, device="cuda")
    t0 = time.perf_counter()
    K.tp_allreduce_tagged(to_torch(part), y, residual=to_torch(res), **link(ranks, 0, n))   # rank 1 never calls
    torch.cuda.synchronize()
    waited = time.perf_counter() - t0
    assert int(ranks[0].status.item()) == -6            # IRON_ERR_TIMEOUT, reported not raised
    assert 1.0 < waited < 10.0
    assert ranks[0].state.tolist()[:2] == [1, 0]        # the kernel ran to its end
    # it went on with what it had: its own rows plus the absent rank's zeros
    want = (part.astype(np.float32) + res.astype(np.float32)).astype(bfloat16)
    assert np.array_equal(to_numpy(y).view(np.uint16), want.view(np.uint16))
