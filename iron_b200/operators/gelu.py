"""GELU (iron/operators/gelu.py:13)."""

import math

import numpy as np

from ..declare import param
from ..elementwise import Sweep, UnaryElementwise
from ..testing import Testing

_erf = np.vectorize(math.erf, otypes=[np.float64])


class GELU(UnaryElementwise):
    """GELU by its tanh approximation, or exact (``approximate="none"``, ``x * Phi(x)``)."""

    test = Testing([Sweep(), Sweep(approximate="none")], draw=lambda op: dict(centered=(op.x,)))

    approximate: str = param(default="tanh", array=True)

    def validate(self) -> None:
        if self.approximate not in ("tanh", "none"):
            raise ValueError(f"GELU: approximate={self.approximate!r} is neither 'tanh' nor 'none'")

    @property
    def ew(self) -> str:
        return "gelu_erf" if self.approximate == "none" else "gelu_tanh"

    def reference(self, x):
        f = x.astype(np.float64)
        if self.approximate == "none":
            y = 0.5 * f * (1.0 + _erf(f / math.sqrt(2.0)))
        else:
            y = 0.5 * f * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (f + 0.044715 * f ** 3)))
        return y.astype(np.float32).astype(x.dtype)
