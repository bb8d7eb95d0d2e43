"""LayerNorm (iron/operators/layer_norm.py:10 on WeightedRowwise, beta 0)."""

import numpy as np

from ..declare import param
from ..elementwise import WeightedRowwise
from ..testing import Case, Testing
from ..verify import Tolerance


class LayerNorm(WeightedRowwise):
    """Each row minus its mean over its (biased) standard deviation, rounded, optionally
    times a learned weight row, rounded again."""

    test = Testing([Case(dict(rows=1, tile_size=2048, weighted=True)),
                    Case(dict(rows=32, tile_size=512)),
                    Case(dict(rows=2048, tile_size=2048, weighted=True), bench=True)],
                   draw=lambda op: dict(centered=(op.x,)))

    epsilon: float = param(default=1e-5, array=True)

    def validate(self):
        if self.tile_size % 8:
            raise ValueError(f"LayerNorm: tile_size ({self.tile_size}) must be a multiple of 8")

    def ops(self) -> int:
        return 5 * self.rows * self.tile_size

    def reference(self, x, weight=None):
        xf = x.astype(np.float32)
        mean = np.mean(xf, axis=-1, keepdims=True, dtype=np.float32)
        d = xf - mean
        inv = np.float32(1.0) / np.sqrt(np.mean(d * d, axis=-1, keepdims=True, dtype=np.float32)
                                        + np.float32(self.epsilon))
        normed = (d * inv).astype(x.dtype)
        if weight is None:
            return normed
        return (normed.astype(np.float32) * weight.astype(np.float32)).astype(x.dtype)

    def tolerance(self):
        return Tolerance.bf16_ulps(1, atol=1e-3, note="f32 arithmetic; the sums' order differs, and near "
                                   "the mean the difference cancels")

    def launch(self, buffers, values):
        from .. import kernels as K

        K.layer_norm(buffers["x"], buffers.get("weight"), buffers["y"], eps=self.epsilon, valid=self.valid)
