"""CausalConv1d: the short depth-wise causal filter of ``F.causal_conv1d`` as one step.

The reference has no operator class for it: ``iron/functional.py:147-180`` records the
filter as a chain of RowwiseMul and ElementwiseAdd steps over a two-block window state, plus
the copies that carry the last ``K - 1`` rows to the next call.  Here one kernel computes
the same chain -- every product and every partial sum rounded to bf16, in the chain's order
-- so the result is bit for bit the recorded steps'.
"""

import numpy as np

from ..declare import In, Operator, Out, param, per_call
from ..testing import Case, Testing
from ..verify import Tolerance


def _bf(a, dtype):
    return a.astype(dtype).astype(np.float32)


class CausalConv1d(Operator):
    """``y[t] = sum_k taps[k] * xx[t + k]``, ``xx`` the ``K - 1`` carried rows then ``x``.

    ``decode`` selects the one-row form's order of the sum (newest tap first, then the
    carried rows oldest first), as the reference's decode branch records it.
    """

    test = Testing([Case(dict(rows=1, channels=256, kernel_size=4, decode=True), id="decode"),
                    Case(dict(rows=7, channels=64, kernel_size=4)),
                    Case(dict(rows=64, channels=512, kernel_size=3)),
                    Case(dict(rows=2, channels=64, kernel_size=4), id="shorter_than_the_carry"),
                    Case(dict(rows=2048, channels=4352, kernel_size=4), bench=True)],
                   draw=lambda op: dict(centered=(op.x, op.taps, op.history)))

    rows: int = param(array=True)
    channels: int = param(array=True)
    kernel_size: int = param(array=True)
    decode: bool = param(default=False)
    carried: int = param(derive=lambda op: op.kernel_size - 1, repr=False)

    x = In(rows, channels)
    taps = In(kernel_size, channels)
    history = In(carried, channels)
    y = Out(rows, channels)
    new_history = Out(carried, channels)
    valid = per_call(bounds=rows)

    def validate(self):
        if self.kernel_size not in (2, 3, 4):
            raise ValueError(f"CausalConv1d: kernel_size ({self.kernel_size}) is 2, 3 or 4")
        if self.channels % 8:
            raise ValueError(f"CausalConv1d: channels ({self.channels}) must be a multiple of 8")
        if self.decode and self.rows != 1:
            raise ValueError(f"CausalConv1d: the decode form takes one row, not {self.rows}")

    def ops(self) -> int:
        return 2 * self.rows * self.channels * self.kernel_size

    def tolerance(self):
        return Tolerance.exact(note="the recorded chain's own roundings, in its order")

    def reference(self, x, taps, history):
        K, n, dt = self.kernel_size, self.valid, x.dtype
        full = np.concatenate([np.asarray(history), np.asarray(x)[:n]], axis=0).astype(np.float32)
        t = np.asarray(taps).astype(np.float32)
        order = [K - 1, *range(K - 1)] if self.decode else list(range(K))
        acc = _bf(full[order[0] : order[0] + n] * t[order[0]], dt)
        for k in order[1:]:
            acc = _bf(acc + _bf(full[k : k + n] * t[k], dt), dt)
        y = np.zeros((self.rows, self.channels), dt)
        y[:n] = acc.astype(dt)
        return y, full[n:].astype(dt)

    def launch(self, buffers, values):
        from .. import kernels as K

        K.causal_conv1d(buffers["x"], buffers["taps"], history=buffers["history"],
                        new_history=buffers["new_history"], out=buffers["y"], valid=self.valid,
                        d_valid=values.get("d_valid"), decode_order=self.decode)
