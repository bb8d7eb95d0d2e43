"""SiLU (iron/operators/silu.py:12)."""

import numpy as np

from ..elementwise import Sweep, UnaryElementwise
from ..testing import Testing


class SiLU(UnaryElementwise):
    """``x * sigmoid(x)`` in float32, rounded once."""

    test = Testing(Sweep(channels=None), draw=lambda op: dict(centered=(op.x,)))
    ew = "silu"

    def reference(self, x):
        f = x.astype(np.float32)
        return (f / (1 + np.exp(-f))).astype(x.dtype)
