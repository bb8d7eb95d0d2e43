"""Sigmoid (iron/operators/sigmoid.py)."""

import numpy as np

from ..elementwise import Sweep, UnaryElementwise
from ..testing import Testing


class Sigmoid(UnaryElementwise):
    """``1 / (1 + exp(-x))`` in float32, rounded once."""

    test = Testing(Sweep(channels=None), draw=lambda op: dict(centered=(op.x,)))
    ew = "sigmoid"

    def reference(self, x):
        f = x.astype(np.float32)
        return (1 / (1 + np.exp(-f))).astype(x.dtype)
