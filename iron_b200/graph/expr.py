"""Per-call integer values as small closed-form expressions.

A graph's per-call values (a position, a row count) may index, bound and offset handles,
but never steer the recording.  As in the reference (``Affine``/``PerCall``, pinned by
iron/tests/common/test_graph.py:534-600 and :898-945) an expression is

    ((scale * v + bias) >> down  [mod 2^k]) * mul + add      [clamped to lo..hi]

in one named value ``v``: closed under ``+ - *`` by ints, ``//`` and ``%`` by powers of
two (nested floors fold), sums of two linear forms in the same value, and ``clamp``.
Anything else -- ``// 3``, ``% 48``, comparisons, truth tests, mixing two values -- raises
``TypeError``, so a value can never pick which steps are recorded.
"""

from __future__ import annotations

import dataclasses
from typing import Mapping


def _pow2(n) -> int | None:
    return n.bit_length() - 1 if isinstance(n, int) and n > 0 and n & (n - 1) == 0 else None


@dataclasses.dataclass(frozen=True, eq=False)
class Expr:
    name: str
    scale: int = 1
    bias: int = 0
    down: int = 0
    mod: int | None = None
    mul: int = 1
    add: int = 0
    lo: int | None = None
    hi: int | None = None

    # ---- classification ----
    @property
    def clamped(self) -> bool:
        return self.lo is not None or self.hi is not None

    @property
    def linear(self) -> bool:
        return self.down == 0 and self.mod is None and not self.clamped

    def _flat(self) -> "Expr":
        """A linear form with mul/add folded into scale/bias."""
        assert self.linear
        return Expr(self.name, self.scale * self.mul, self.bias * self.mul + self.add)

    # ---- evaluation ----
    def evaluate(self, values: Mapping[str, int]) -> int:
        if self.name not in values:
            raise TypeError(f"per-call value {self.name!r} was not given")
        x = self.scale * int(values[self.name]) + self.bias
        x >>= self.down
        if self.mod is not None:
            x %= self.mod
        x = x * self.mul + self.add
        if self.lo is not None:
            x = max(x, self.lo)
        if self.hi is not None:
            x = min(x, self.hi)
        return x

    # ---- arithmetic ----
    def _refuse(self, what: str):
        raise TypeError(f"{what} is not computed per call: {self.name} is a per call value")

    def __add__(self, other):
        if isinstance(other, Expr):
            if other.name != self.name or not (self.linear and other.linear):
                self._refuse("a sum of two per-call forms that are not linear in one value")
            a, b = self._flat(), other._flat()
            return Expr(self.name, a.scale + b.scale, a.bias + b.bias)
        if not isinstance(other, int):
            return NotImplemented
        if self.clamped:
            self._refuse("arithmetic on a clamped value")
        return dataclasses.replace(self, add=self.add + other)

    __radd__ = __add__

    def __sub__(self, other):
        if isinstance(other, Expr):
            return self + (other * -1)
        if not isinstance(other, int):
            return NotImplemented
        return self + (-other)

    def __rsub__(self, other):
        return (self * -1) + other

    def __mul__(self, other):
        if not isinstance(other, int):
            if isinstance(other, Expr):
                self._refuse("a product of two per-call values")
            return NotImplemented
        if self.clamped:
            self._refuse("arithmetic on a clamped value")
        return dataclasses.replace(self, mul=self.mul * other, add=self.add * other)

    __rmul__ = __mul__

    def __floordiv__(self, other):
        k = _pow2(other)
        if k is None or self.clamped or self.mod is not None:
            self._refuse(f"// {other}")
        if self.mul == 1 and self.add == 0:
            return dataclasses.replace(self, down=self.down + k)
        if self.down == 0:
            f = self._flat()
            return Expr(self.name, f.scale, f.bias, down=k)
        self._refuse(f"// {other} of a scaled floor")

    def __mod__(self, other):
        k = _pow2(other)
        if k is None or self.clamped or self.mod is not None:
            self._refuse(f"% {other}")
        if self.mul == 1 and self.add == 0:
            return dataclasses.replace(self, mod=other)
        if self.down == 0:
            f = self._flat()
            return Expr(self.name, f.scale, f.bias, mod=other)
        self._refuse(f"% {other} of a scaled floor")

    def clamp(self, lo: int | None = None, hi: int | None = None) -> "Expr":
        return dataclasses.replace(self, lo=lo if self.lo is None else max(self.lo, lo or self.lo),
                                   hi=hi if self.hi is None else min(self.hi, hi or self.hi))

    def difference(self, other) -> int | None:
        """``self - other`` when it is the same for every call, else None."""
        if isinstance(other, int):
            return None
        if other.name != self.name or not (self.linear and other.linear):
            return None
        a, b = self._flat(), other._flat()
        return a.bias - b.bias if a.scale == b.scale else None

    # ---- never steers the recording ----
    def __bool__(self):
        self._refuse("a truth test")

    def _compare(self, other):
        self._refuse("a comparison")

    __lt__ = __le__ = __gt__ = __ge__ = _compare

    def __eq__(self, other):
        if isinstance(other, Expr):
            return dataclasses.astuple(self) == dataclasses.astuple(other)
        self._refuse("a comparison")

    def __hash__(self):
        return hash(dataclasses.astuple(self))

    def __index__(self):
        self._refuse("use as a Python integer")

    def __repr__(self):
        return (f"Expr({self.name}: (({self.scale}v+{self.bias})>>{self.down}"
                f"{'' if self.mod is None else f' % {self.mod}'})*{self.mul}+{self.add}"
                f"{f' in [{self.lo},{self.hi}]' if self.clamped else ''})")


def clamp(value, lo: int | None = None, hi: int | None = None):
    """``value`` held within ``lo..hi`` (iron.clamp)."""
    if isinstance(value, Expr):
        return value.clamp(lo, hi)
    v = int(value)
    if lo is not None:
        v = max(v, lo)
    if hi is not None:
        v = min(v, hi)
    return v


def evaluate(value, values: Mapping[str, int]) -> int:
    return value.evaluate(values) if isinstance(value, Expr) else int(value)
