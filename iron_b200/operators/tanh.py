"""Tanh (iron/operators/tanh.py:9)."""

import numpy as np

from ..elementwise import Sweep, UnaryElementwise
from ..testing import Testing


class Tanh(UnaryElementwise):
    """``tanh(x)`` in float32, rounded once.

    The reference's device kernel is a table lookup up to 0.0051 off ``tanh``; here the
    float32 function itself is computed, so the result is the rounding of the true value.
    """

    test = Testing(Sweep(), draw=lambda op: dict(centered=(op.x,)))
    ew = "tanh"

    def reference(self, x):
        return np.tanh(x.astype(np.float32)).astype(x.dtype)
