"""AXPY (iron/operators/axpy.py:12)."""

import numpy as np

from ..declare import param
from ..elementwise import BinaryElementwise, Sweep
from ..testing import Case, Testing


class AXPY(BinaryElementwise):
    """``scalar_factor * a + b``."""

    test = Testing([Sweep(channels=None, scalar_factor=3.0), Case(dict(size=2048, scalar_factor=1.003))],
                   draw=lambda op: dict(centered=(op.a, op.b)))
    ew = "axpy"

    scalar_factor: float = param(default=3.0, array=True)

    def scalars(self):
        return (self.scalar_factor,)

    def reference(self, a, b):
        return (np.float32(self.scalar_factor) * a.astype(np.float32) + b.astype(np.float32)).astype(a.dtype)
