"""ReLU (iron/operators/relu.py:11)."""

import numpy as np

from ..elementwise import Sweep, UnaryElementwise
from ..testing import Testing


class ReLU(UnaryElementwise):
    """``max(x, 0)``: exact in bf16."""

    test = Testing(Sweep(), draw=lambda op: dict(centered=(op.x,)))  # both signs
    ew = "relu"

    def reference(self, x):
        return np.maximum(x.astype(np.float32), np.float32(0)).astype(x.dtype)
