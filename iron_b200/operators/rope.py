"""RoPE (iron/operators/rope.py:58)."""

import numpy as np
from ml_dtypes import bfloat16

from ..declare import In, Operator, Out, param, per_call, tunable
from ..testing import Case, Testing
from ..verify import Tolerance


def _angles(op):
    """A random angle table, cos and sin interleaved, a row per position (rope.py:48-55)."""
    rng = np.random.default_rng(0)
    theta = rng.uniform(-np.pi, np.pi, (op.angle_rows, op.cols // 2))
    table = np.empty((op.angle_rows, op.cols), dtype=np.float32)
    table[:, ::2], table[:, 1::2] = np.cos(theta), np.sin(theta)
    return dict(given={op.angles: table.astype(bfloat16)})


class RoPE(Operator):
    """Rotate each row of ``x`` by its angle row; each angle row serves ``rows / angle_rows`` rows."""

    test = Testing([Case(dict(rows=32, cols=512, angle_rows=8)), Case(dict(rows=32, cols=512, angle_rows=32)),
                    Case(dict(rows=32, cols=128, angle_rows=8, two_halves=False)),
                    Case(dict(rows=64, cols=128, angle_rows=16), extensive=True),
                    Case(dict(rows=4096, cols=512, angle_rows=8), bench=True)], draw=_angles)

    rows: int = param()
    cols: int = param()
    angle_rows: int = param(default=lambda op: op.rows)
    num_aie_columns: int = tunable()
    two_halves: bool = param(default=True, array=True)

    x = In(rows, cols)
    angles = In(angle_rows, cols)
    y = Out(rows, cols)
    valid = per_call(bounds=rows)
    valid_angles = per_call(bounds=angle_rows)

    def validate(self):
        if not (self.cols % 32 == 0 and self.cols >= 32):
            raise ValueError(f"RoPE: cols ({self.cols}) must be a positive multiple of 32")
        if not (self.angle_rows <= self.rows and self.rows % self.angle_rows == 0):
            raise ValueError(f"RoPE: angle_rows ({self.angle_rows}) must divide rows ({self.rows})")

    def ops(self) -> int:
        return 3 * self.rows * self.cols

    def reference(self, x, angles):
        rows, cols, lut = x.shape[0], x.shape[-1], angles.shape[0]
        if rows % lut:
            raise ValueError(f"RoPE: angles ({lut} rows) must divide x's {rows} rows")
        xr = x.astype(np.float32).reshape(lut, -1, cols)
        cos = angles[:, 0::2].astype(np.float32).reshape(lut, 1, cols // 2)
        sin = angles[:, 1::2].astype(np.float32).reshape(lut, 1, cols // 2)
        out = np.empty_like(xr)
        if self.two_halves:
            h = cols // 2
            out[..., :h] = xr[..., :h] * cos - xr[..., h:] * sin
            out[..., h:] = xr[..., h:] * cos + xr[..., :h] * sin
        else:
            out[..., 0::2] = xr[..., 0::2] * cos - xr[..., 1::2] * sin
            out[..., 1::2] = xr[..., 1::2] * cos + xr[..., 0::2] * sin
        return out.reshape(x.shape).astype(x.dtype)

    def tolerance(self):
        return Tolerance.relative(0.05, note="bit-exact with the reference formula on bf16 tables")

    def launch(self, buffers, values):
        from .. import kernels as K

        K.rope(buffers["x"], buffers["angles"], buffers["y"], angle_rows=self.angle_rows,
               two_halves=self.two_halves, valid=self.valid)
