"""Helpers shared by the tests: bf16 numpy <-> torch, seeded draws, judging."""

import numpy as np
from ml_dtypes import bfloat16


def to_torch(a: np.ndarray, device="cuda"):
    """A numpy array (bf16 via ml_dtypes included) as a torch tensor on ``device``."""
    import torch

    a = np.ascontiguousarray(a)
    if a.dtype == bfloat16:
        return torch.from_numpy(a.view(np.int16)).view(torch.bfloat16).to(device)
    return torch.from_numpy(a).to(device)


def to_numpy(t) -> np.ndarray:
    """A torch tensor as numpy, bf16 kept as ml_dtypes' bfloat16."""
    import torch

    t = t.detach().cpu().contiguous()
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy().view(bfloat16)
    return t.numpy()


def normal(rng, shape, scale=1.0, dtype=bfloat16):
    return (rng.standard_normal(shape, dtype=np.float32) * np.float32(scale)).astype(dtype)


def assert_verdict(got, want, tolerance, bound=None, what=""):
    from iron_b200.verify import compare

    v = compare(got, want, tolerance, bound=bound)
    assert v, f"{what}: {v.detail}"


def assert_bf16_bound(got, want, what=""):
    """The bound every bf16 output is held to: within 1e-2 relative or 2e-2 absolute."""
    g = np.asarray(got).astype(np.float64)
    w = np.asarray(want).astype(np.float64)
    err = np.abs(g - w)
    ok = (err <= 1e-2 * np.abs(w)) | (err <= 2e-2)
    assert ok.all(), f"{what}: {int((~ok).sum())}/{ok.size} beyond 1e-2 rel / 2e-2 abs; max err {err.max():.4g}"


def fast_random_weights(named: dict, seed: int) -> dict:
    """``oracle.model.filled_random``'s draw with the bf16 rounding done by torch (the same
    round-to-nearest-even, many times faster on 100-million-element embeddings)."""
    import math

    import torch

    rng = np.random.default_rng(seed)
    out = {}
    for n, shape in named.items():
        x = rng.standard_normal(shape, dtype=np.float32)
        if len(shape) >= 2:
            x /= np.float32(np.sqrt(math.prod(shape[1:])))
        else:
            x = x / 10 + (not n.endswith("bias"))
        out[n] = torch.from_numpy(np.ascontiguousarray(x, np.float32)).to(torch.bfloat16).view(torch.int16).numpy().view(bfloat16)
    return out
