"""Clamp (iron/operators/clamp.py:16)."""

import numpy as np

from ..declare import param
from ..elementwise import Sweep, UnaryElementwise
from ..testing import Case, Testing
from ..verify import Tolerance


class Clamp(UnaryElementwise):
    """``x`` clamped to ``[low, high]``, elementwise, the bounds rounded to bf16."""

    test = Testing([Sweep(low=-0.75, high=1.25),
                    # bounds of one sign, and one past every input: the identity
                    Case(dict(size=2048, low=0.5, high=1.5)),
                    Case(dict(size=2048, low=-3e4, high=3e4))],
                   draw=lambda op: dict(centered=(op.x,)))

    low: float = param()
    high: float = param()

    def validate(self) -> None:
        if not np.float32(self.low) <= np.float32(self.high):
            raise ValueError(f"Clamp: low ({self.low}) exceeds high ({self.high})")

    def reference(self, x):
        lo, hi = (np.array(b, x.dtype).astype(np.float32) for b in (self.low, self.high))
        return np.minimum(np.maximum(x.astype(np.float32), lo), hi).astype(x.dtype)

    def tolerance(self):
        return Tolerance.exact(note="a selection among bf16 values")

    def launch(self, buffers, values):
        from .. import kernels as K

        K.clamp(buffers["x"].view(-1)[: self.valid], self.low, self.high, buffers["y"].view(-1)[: self.valid])
