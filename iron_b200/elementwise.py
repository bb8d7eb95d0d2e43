"""Templates shared by the unary, binary, row-wise and row-broadcast operators.

The host half of ``iron/common/elementwise.py`` (``Elementwise`` :151, ``UnaryElementwise``
:494, ``BinaryElementwise`` :525, ``Rowwise`` :555, ``WeightedRowwise`` :619,
``RowBroadcast`` :797, ``Sweep`` :44): the same field and operand names; the device half is
one launch of the element-wise / row-wise kernels.
"""

from __future__ import annotations

import numpy as np

from .declare import In, Operator, Out, param, per_call, tunable
from .testing import Case
from .verify import Tolerance


class Sweep:
    """The default case list of an element-wise operator: a few sizes, one benchmarked."""

    def __init__(self, channels=None, **extra):
        self.extra = extra

    def __call__(self, cls, dev=None):
        sizes = [2048, 8192, 65536]
        if issubclass(cls, Rowwise):
            return [Case(dict(rows=r, tile_size=t, **self.extra), bench=(r * t >= 2 ** 20))
                    for r, t in ((1, 2048), (32, 512), (2048, 2048))]
        return [Case(dict(size=s, **self.extra), bench=(s == sizes[-1])) for s in sizes]


class Elementwise(Operator):
    num_aie_columns: int = tunable()
    num_channels: int = tunable(default=1)

    #: name of the element-wise kernel op (see ``iron_b200.kernels.EW``)
    ew: str = ""

    def ops(self) -> int:
        return int(np.prod(self.outputs[0].shape))


class UnaryElementwise(Elementwise):
    size: int = param()
    tile_size: int = tunable()
    valid = per_call(bounds=size)

    x = In(size)
    y = Out(size)

    def launch(self, buffers, values):
        from . import kernels as K

        K.elementwise(self.ew, buffers["x"].view(-1)[: self.valid], None, buffers["y"].view(-1)[: self.valid])

    def tolerance(self):
        return Tolerance.bf16_ulps(1, note="f32 arithmetic, rounded once")


class BinaryElementwise(Elementwise):
    size: int = param()
    tile_size: int = tunable()
    valid = per_call(bounds=size)

    a = In(size)
    b = In(size)
    y = Out(size)

    def scalars(self) -> tuple:
        return ()

    def launch(self, buffers, values):
        from . import kernels as K

        n = self.valid
        s = self.scalars()
        K.elementwise(self.ew, buffers["a"].view(-1)[:n], buffers["b"].view(-1)[:n], buffers["y"].view(-1)[:n],
                      scalar=s[0] if s else 0.0)

    def tolerance(self):
        return Tolerance.bf16_ulps(1, note="f32 arithmetic, rounded once")


class Rowwise(Elementwise):
    rows: int = param()
    tile_size: int = param(array=True)
    valid = per_call(bounds=rows)

    x = In(rows, tile_size)
    y = Out(rows, tile_size)


class WeightedRowwise(Rowwise):
    weighted: bool = param(default=False)

    x = In("rows", "tile_size")
    weight = In("tile_size", when=weighted)
    y = Out("rows", "tile_size")


class RowBroadcast(Rowwise):
    x = In("rows", "tile_size")
    row = In("tile_size")
    y = Out("rows", "tile_size")

    def launch(self, buffers, values):
        from . import kernels as K

        n = self.valid
        K.elementwise(self.ew, buffers["x"][:n], buffers["row"], buffers["y"][:n])

    def tolerance(self):
        return Tolerance.bf16_ulps(1, note="f32 arithmetic, rounded once")
