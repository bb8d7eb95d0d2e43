"""The output stage a projection GEMM folds in (iron/operators/flm/gemm/design.py:75-112)."""

from enum import StrEnum

import numpy as np


def _sigmoid(x):
    """``1 / (1 + exp(-x))`` in float32, rounded once back to ``x``'s dtype."""
    f = x.astype(np.float32)
    return (1 / (1 + np.exp(-f))).astype(x.dtype)


class Epilogue(StrEnum):
    NONE = "none"
    GELU = "gelu"
    SILU = "silu"
    SIGMOID = "sigmoid"

    @property
    def mode(self) -> int:
        return list(Epilogue).index(self)

    def apply(self, C):
        """This stage alone on an already-rounded product ``C``."""
        if self is Epilogue.GELU:
            return C * _sigmoid(np.float32(1.702) * C)
        if self is Epilogue.SILU:
            return C * _sigmoid(C)
        if self is Epilogue.SIGMOID:
            return _sigmoid(C)
        return C
