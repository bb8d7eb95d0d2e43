"""Softmax (iron/operators/softmax.py:77)."""

from typing import Any

import numpy as np
from ml_dtypes import bfloat16

from ..declare import In, Operator, Out, param, per_call, tunable
from ..testing import Case, Testing
from ..verify import Tolerance


def _draw(op) -> dict:
    """The float32 path's logits and addend centred; the bf16 path draws ``[0, scale)``."""
    if np.dtype(op.input_dtype) != np.dtype(np.float32):
        return {}
    return dict(centered=(op.x,) + ((op.addend,) if op.has_addend else ()))


class Softmax(Operator):
    """Softmax over each row's first ``length`` columns; the columns past them are zeros.

    The float32 input path takes a pre-cap addend and a soft cap ``cap * tanh(x / cap)``
    (iron/operators/softmax.py:129-133).  Its banded form (``window``, ``period``) computes a
    mask whose definition lives outside the reference tree; it is refused here.
    """

    test = Testing([Case(dict(rows=32, cols=1024)),
                    Case(dict(rows=16, cols=4096)),
                    Case(dict(rows=16, cols=4608)),
                    Case(dict(rows=32, cols=32768)),
                    Case(dict(rows=4096, cols=512), bench=True),
                    Case(dict(rows=32, cols=1024, input_dtype=np.float32)),
                    Case(dict(rows=64, cols=32, input_dtype=np.float32, soft_cap=50.0, has_addend=True),
                         id="f32_soft_cap_addend")],
                   draw=_draw)

    rows: int = param(array=True)
    cols: int = param()
    num_aie_columns: int = tunable()
    num_channels: int = tunable(default=1)
    block: int = tunable()
    streamed: bool = tunable()
    input_dtype: Any = param(default=bfloat16, repr=False)
    soft_cap: float | None = param(default=None, array=True)
    has_addend: bool = param(default=False)
    window: int | None = param(default=None, array=True)
    period: int | None = param(default=None, array=True)

    length = per_call(bounds=cols)  # cols, or fewer per call

    x = In(rows, cols, dtype=input_dtype)
    addend = In(rows, cols, dtype=np.float32, when=has_addend)
    y = Out(rows, cols)

    def validate(self) -> None:
        if self.rows % 16 != 0:
            raise ValueError(f"Softmax: rows ({self.rows}) must be a multiple of 16")
        if self.cols % 16 != 0:
            raise ValueError(f"Softmax: cols ({self.cols}) must be a multiple of 16")
        f32 = np.dtype(self.input_dtype) == np.dtype(np.float32)
        if not f32 and np.dtype(self.input_dtype) != np.dtype(bfloat16):
            raise ValueError(f"Softmax: input_dtype ({self.input_dtype}) is bfloat16 or float32")
        if not f32 and (self.soft_cap is not None or self.has_addend or self.window is not None
                        or self.period is not None):
            raise ValueError("Softmax: soft_cap, addend, window and period are options "
                             "of the float32 input path; pass input_dtype=np.float32")
        if (self.window is None) != (self.period is None):
            raise ValueError("Softmax: window and period are given together")
        if self.window is not None:
            raise NotImplementedError("Softmax: the banded path (window, period) is not provided")
        if self.soft_cap is not None and not self.soft_cap > 0:
            raise ValueError(f"Softmax: soft_cap ({self.soft_cap}) must be positive")

    def ops(self) -> int:
        return 4 * self.rows * self.cols

    def tolerance(self):
        return Tolerance.bf16_ulps(1, atol=1e-6, note="f32 throughout, y rounded once; the sum's order differs")

    def reference(self, x, *rest):
        n = self.length
        v = np.asarray(x)[..., :n].astype(np.float32)
        if self.has_addend:
            v = v + np.asarray(rest[0])[..., :n].astype(np.float32)
        if self.soft_cap is not None:
            v = np.float32(self.soft_cap) * np.tanh(v / np.float32(self.soft_cap))
        out = np.zeros((self.rows, self.cols), bfloat16)
        if n:
            e = np.exp(v - v.max(axis=-1, keepdims=True))
            out[..., :n] = (e / e.sum(axis=-1, keepdims=True, dtype=np.float32)).astype(bfloat16)
        return out

    def launch(self, buffers, values):
        from .. import kernels as K

        K.softmax(buffers["x"], buffers["y"], addend=buffers.get("addend"), soft_cap=self.soft_cap,
                  length=self.length, d_length=values.get("d_length"))
