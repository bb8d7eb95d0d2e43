"""A decode step's attention + o_proj + residual add in one launch (after the fused q/k/v
kernel) against the chain of operator references (B200): RMSNorm, q/k/v GEMVs, RoPE, the
cache writes, one-query attention with grouped heads, o_proj and the residual add
(iron/lm/blocks.py:627-648, :472-502, :723-728), every operator rounding to bf16 as the
oracle's restatements do, and against the two separate kernels it replaces.
"""

import numpy as np
import pytest
from ml_dtypes import bfloat16

from oracle import ops
from oracle.model import rope_angles
from tests.util import assert_bf16_bound, normal, to_numpy, to_torch

pytestmark = pytest.mark.gpu


def chain(x, w, angles, kc, vc, pos, H, G, D, window=None, scale=None, eps=1e-5):
    """The reference's recorded steps on the host; returns (y, k row, v row)."""
    h = ops.rms_norm(x[None], w["norm"], eps)[0]
    qkv = ops.gemv(w["qkv"], h)
    q, k, v = qkv[: H * D].reshape(H, D), qkv[H * D : (H + G) * D].reshape(G, D), qkv[(H + G) * D :].reshape(G, D)
    q, k = ops.rope(q, angles[pos : pos + 1]), ops.rope(k, angles[pos : pos + 1])
    kc, vc = kc.copy(), vc.copy()
    kc[pos], vc[pos] = k, v
    o = ops.mha(q[None], kc[: pos + 1], vc[: pos + 1], num_heads=H, num_kv_heads=G, heads_interleaved=True,
                kv_interleaved=True, window=window, scale=scale).reshape(H * D)
    return ops.add(x, ops.gemv(w["o"], o)), k, v


CASES = [
    # E, H, G, D, cache rows, position, window
    (2048, 32, 8, 64, 2304, 0, None),
    (2048, 32, 8, 64, 2304, 5, None),
    (2048, 32, 8, 64, 2304, 2100, None),
    (2048, 32, 8, 64, 4096, 3500, None),     # more keys per CTA than one shared-memory pass holds
    (2048, 32, 8, 64, 4096, 2303, None),
    (2048, 32, 8, 64, 2304, 2047, 511),
    (512, 16, 4, 64, 256, 200, None),        # the toy decoder's shape
    (1024, 8, 4, 128, 512, 300, None),       # 128-wide heads, two query heads a group
    (512, 4, 4, 64, 128, 77, None),          # one query head a group
]


@pytest.mark.parametrize("E,H,G,D,S,pos,window", CASES)
def test_attention_and_o_proj_in_one_launch_match_the_operator_chain(E, H, G, D, S, pos, window):
    import torch

    from iron_b200 import kernels as K

    assert K.attn_oproj_supported(E, H, G, D) >= 32
    rng = np.random.default_rng(E + pos)
    x = normal(rng, (E,))
    w = {"norm": (1 + rng.standard_normal(E) / 10).astype(bfloat16),
         "qkv": normal(rng, ((H + 2 * G) * D, E), 1 / np.sqrt(E)),
         "o": normal(rng, (E, H * D), 1 / np.sqrt(H * D))}
    angles = rope_angles(D, S, 500000.0).astype(bfloat16)
    kc, vc = normal(rng, (S, G, D)), normal(rng, (S, G, D))
    want, wk, wv = chain(x, w, angles, kc, vc, pos, H, G, D, window=window)
    d = {k: to_torch(v) for k, v in w.items()}
    tx, tk, tv = to_torch(x), to_torch(kc), to_torch(vc)
    q = torch.empty(1, H, D, dtype=torch.bfloat16, device="cuda")
    y = torch.empty(E, dtype=torch.bfloat16, device="cuda")
    scratch = K.attn_oproj_scratch(E, G, "cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    dpos = torch.tensor([pos], dtype=torch.int32, device="cuda")
    for _ in range(2):   # the scratch's counters are left ready for the next launch
        K.decode_qkv_rope(d["qkv"], tx, to_torch(angles), tk, tv, q[0], H=H, G=G, D=D, d_position=dpos,
                          norm_weight=d["norm"])
        K.decode_attn_oproj(q[0], d["o"], tx, tk, tv, y, G=G, scratch=scratch, d_position=dpos, window=window,
                            status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    assert_bf16_bound(to_numpy(y), want, "y")
    assert_bf16_bound(to_numpy(tk[pos]), wk, "k row")
    assert_bf16_bound(to_numpy(tv[pos]), wv, "v row")
    # and it is what the two separate kernels give, within the same bound
    att = torch.empty(1, H, D, dtype=torch.bfloat16, device="cuda")
    K.mha_decode(q, tk[None], tv[None], att, kv_valid=pos + 1, window=window)
    y2 = K.gemv(d["o"], att.view(-1), residual=tx)
    assert_bf16_bound(to_numpy(y), to_numpy(y2).astype(np.float32), "against the separate kernels")


def test_shapes_whose_rows_do_not_fit_an_sm_are_refused_on_the_host():
    import torch

    from iron_b200 import _lib, kernels as K

    assert K.attn_oproj_supported(3072, 24, 8, 128) == 0      # the 3B shape: three 128-wide heads a group
    assert K.attn_oproj_supported(4096, 32, 8, 128) == 0      # four 128-wide heads a group
    assert K.attn_oproj_supported(2048, 32, 16, 64) == 0      # more groups than clusters resident at once
    z = torch.zeros(64, dtype=torch.bfloat16, device="cuda")
    rc = _lib.load().iron_decode_attn_oproj_bf16(z.data_ptr(), z.data_ptr(), z.data_ptr(), 0, None, z.data_ptr(),
                                                 z.data_ptr(), z.data_ptr(), 3072, 24, 8, 128, 16, -1, 1.0,
                                                 z.data_ptr(), None, None)
    assert rc == -4   # IRON_ERR_UNSUPPORTED: nothing launched
