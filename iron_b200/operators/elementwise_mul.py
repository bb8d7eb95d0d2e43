"""ElementwiseMul and RowwiseMul (iron/operators/elementwise_mul.py:11,18)."""

import numpy as np

from ..elementwise import BinaryElementwise, RowBroadcast, Sweep
from ..testing import Testing


class ElementwiseMul(BinaryElementwise):
    """``a * b``: SwiGLU's product."""

    test = Testing(Sweep(channels=None), draw=lambda op: dict(centered=(op.a, op.b)))
    ew = "mul"

    def reference(self, a, b):
        return (a.astype(np.float32) * b.astype(np.float32)).astype(a.dtype)


class RowwiseMul(RowBroadcast):
    """Each row times one row."""

    test = Testing(Sweep(channels=None), draw=lambda op: dict(centered=(op.x, op.row)))
    ew = "row_mul"

    def reference(self, x, row):
        return (x.astype(np.float32) * row.astype(np.float32)).astype(x.dtype)
