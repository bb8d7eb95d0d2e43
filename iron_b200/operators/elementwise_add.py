"""ElementwiseAdd and RowwiseAdd (iron/operators/elementwise_add.py:11,18)."""

import numpy as np

from ..elementwise import BinaryElementwise, RowBroadcast, Sweep
from ..testing import Testing


class ElementwiseAdd(BinaryElementwise):
    """``a + b``: the residual add."""

    test = Testing(Sweep(channels=None), draw=lambda op: dict(centered=(op.a, op.b)))
    ew = "add"

    def reference(self, a, b):
        return (a.astype(np.float32) + b.astype(np.float32)).astype(a.dtype)


class RowwiseAdd(RowBroadcast):
    """Each row plus one row: a projection's bias."""

    test = Testing(Sweep(channels=None), draw=lambda op: dict(centered=(op.x, op.row)))
    ew = "row_add"

    def reference(self, x, row):
        return (x.astype(np.float32) + row.astype(np.float32)).astype(x.dtype)
