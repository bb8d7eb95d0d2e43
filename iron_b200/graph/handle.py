"""Handles: what a graph's body computes with.

A ``Handle`` is a contiguous row-major view of a buffer: an element offset (an int, or a
per-call ``Expr`` when the body indexed by a per-call value), a shape, and an optional
per-call bound on its leading axis (``x[:n]``).  Indexing, slicing the leading axis,
reshaping and arithmetic record nothing until an operator consumes the view; assignment
into a view and arithmetic record steps on the active recorder.  This is the contract of
``iron/common/graph/handle.py:95-602`` for the forms the decoder path uses (the
body expressions: ``cache[position] = k``, ``cache[start:start+C][:rows] = x``,
``keys[:position+1]``, ``table[position]``, ``embed[ids]``, ``w[a:b]``, ``x[rows-1]``,
reshapes carrying the leading bound, ``x + y``, ``x * w``, ``x - y``).

Held objects -- ``param`` (a checkpoint weight), ``weight`` (a constant array) and ``state``
(device memory that persists between calls) -- become handles when a body touches them.
"""

from __future__ import annotations

import dataclasses
import math
from fractions import Fraction
from typing import Any

import numpy as np
from ml_dtypes import bfloat16

from ..declare import graph_recorder
from .expr import Expr


@dataclasses.dataclass(eq=False)
class BufferRef:
    """One buffer of a recording: an input, a resident (weight/state) or a transient."""

    kind: str                 # "input" | "weight" | "state" | "transient"
    name: str
    shape: tuple[int, ...]
    dtype: Any
    held: Any = None          # the Param / Weight / State behind a resident

    @property
    def elements(self) -> int:
        return int(math.prod(self.shape))

    @property
    def nbytes(self) -> int:
        return self.elements * np.dtype(self.dtype).itemsize


class Held:
    """Base of what a graph holds between calls."""

    shape: tuple[int, ...]
    dtype: Any

    def _handle(self) -> "Handle":
        rec = graph_recorder.get()
        if rec is None:
            raise TypeError(f"{type(self).__name__} is read inside a Graph's body")
        return rec.handle_of(self)

    def __getitem__(self, index):
        return self._handle()[index]

    def __setitem__(self, index, value):
        self._handle()[index] = value

    def reshape(self, *shape):
        return self._handle().reshape(*shape)


class Param(Held):
    """A checkpoint weight: a shape until ``load_state_dict`` binds its array."""

    def __init__(self, *shape_or_array, dtype=bfloat16):
        if len(shape_or_array) == 1 and isinstance(shape_or_array[0], np.ndarray):
            self.array = np.ascontiguousarray(shape_or_array[0])
            self.shape, self.dtype = tuple(self.array.shape), self.array.dtype
        else:
            self.array = None
            self.shape, self.dtype = tuple(int(s) for s in shape_or_array), dtype

    def __array__(self, dtype=None, copy=None):
        if self.array is None:
            raise TypeError("this param was never loaded")
        return self.array if dtype is None else self.array.astype(dtype)

    def astype(self, dtype):
        return np.asarray(self).astype(dtype)

    # Outside a body a loaded param computes as its array (a model folds a scalar into a norm's
    # weight as it loads); with a handle the handle's own arithmetic records a step.
    def _numeric(self, other, fn):
        if isinstance(other, Handle):
            return NotImplemented
        return fn(np.asarray(self), np.asarray(other) if isinstance(other, Held) else other)

    def __truediv__(self, other):
        return self._numeric(other, lambda a, b: a / b)

    def __mul__(self, other):
        return self._numeric(other, lambda a, b: a * b)

    __rmul__ = __mul__

    def __add__(self, other):
        return self._numeric(other, lambda a, b: a + b)

    __radd__ = __add__

    def __sub__(self, other):
        return self._numeric(other, lambda a, b: a - b)

    def __neg__(self):
        return -np.asarray(self)


class Weight(Held):
    """A constant array a graph computes with (a RoPE table)."""

    def __init__(self, array: np.ndarray):
        self.array = np.ascontiguousarray(array)
        self.shape, self.dtype = tuple(self.array.shape), self.array.dtype


class State(Held):
    """Device memory that persists between calls (a KV cache); zeros until written."""

    def __init__(self, shape, dtype=bfloat16, name: str | None = None):
        self.shape, self.dtype, self.name = tuple(int(s) for s in shape), dtype, name
        self.host: np.ndarray | None = None  # the reference path's copy


def param(*shape_or_array, dtype=bfloat16) -> Param:
    return Param(*shape_or_array, dtype=dtype)


def weight(array) -> Weight | Held:
    return array if isinstance(array, Held) else Weight(np.asarray(array))


def state(shape, dtype=bfloat16) -> State:
    return State(shape, dtype)


@dataclasses.dataclass(eq=False)
class Handle:
    """A contiguous view of a buffer (see the module docstring)."""

    buffer: BufferRef
    shape: tuple[int, ...]
    offset: Any = 0                     # elements; int or Expr
    bound: Any = None                   # valid leading rows: int or Expr, in base rows
    per: Fraction = Fraction(1)         # current leading rows per base row of the bound
    ids: "Handle | None" = None         # set on a gather view: rows picked by these ids

    # ---- facts ----
    @property
    def dtype(self):
        return self.buffer.dtype

    @property
    def elements(self) -> int:
        return int(math.prod(self.shape))

    @property
    def valid(self) -> dict:
        """The per-call bound by axis (only the leading axis can carry one)."""
        return {} if self.bound is None else {0: self.rows_bound()}

    def rows_bound(self):
        """The bound in rows of this view's leading axis."""
        if self.bound is None:
            return None
        if self.per == 1:
            return self.bound
        num, den = self.per.numerator, self.per.denominator
        if den == 1:
            return self.bound * num
        # rows merged earlier (n*G rows of D) and split again (n rows of G*D): divide exactly
        b = self.bound
        if isinstance(b, int) and (b * num) % den == 0:
            return b * num // den
        if isinstance(b, Expr) and not b.clamped and b.mod is None and (b.mul * num) % den == 0 \
                and (b.add * num) % den == 0:
            return dataclasses.replace(b, mul=b.mul * num // den, add=b.add * num // den)
        raise TypeError("a bound does not divide into this view's rows")

    def _rec(self):
        rec = graph_recorder.get()
        if rec is None:
            raise TypeError("handles compute inside a Graph's body")
        return rec

    # ---- views ----
    def reshape(self, *shape) -> "Handle":
        if len(shape) == 1 and isinstance(shape[0], (tuple, list)):
            shape = tuple(shape[0])
        shape = tuple(int(s) for s in shape)
        if math.prod(shape) != self.elements:
            raise ValueError(f"cannot reshape {self.shape} to {shape}")
        per = self.per
        if self.bound is not None:
            if not self.shape or not shape:
                raise TypeError("a bounded view keeps a leading axis")
            per = self.per * Fraction(shape[0], self.shape[0])
        return dataclasses.replace(self, shape=shape, per=per)

    def __getitem__(self, index) -> "Handle":
        if isinstance(index, Handle):
            if len(index.shape) != 1:
                raise TypeError("rows are gathered by a vector of ids")
            return dataclasses.replace(self, shape=(index.shape[0], *self.shape[1:]), ids=index,
                                       bound=index.bound, per=index.per)
        if isinstance(index, tuple):
            if all(isinstance(i, slice) and i == slice(None) for i in index[1:]):
                index = index[0]
            else:
                raise TypeError("only the leading axis is indexed or sliced; copy a column block with Copy")
        if not self.shape:
            raise IndexError("a scalar view has no axis to index")
        row = int(math.prod(self.shape[1:]))
        n = self.shape[0]
        if isinstance(index, slice):
            if index.step not in (None, 1):
                raise TypeError("strided slices are not views")
            start, stop = index.start, index.stop
            if start is None and isinstance(stop, Expr):
                # x[:n] by a per-call value: a bound, not a smaller view (a static x[:8] is a slice)
                if isinstance(stop, Expr) and not (stop.linear or stop.clamped):
                    raise TypeError("a bound is linear or clamped per call")
                if self.bound is not None:
                    raise TypeError("the view is already bounded")
                return dataclasses.replace(self, bound=stop, per=Fraction(1))
            start = 0 if start is None else start
            stop = n if stop is None else stop
            if isinstance(start, Expr) or isinstance(stop, Expr):
                width = stop.difference(start) if isinstance(stop, Expr) else None
                if width is None or width <= 0 or width > n:
                    raise TypeError("a per-call slice is a fixed-width run from a per-call start")
                if self.bound is not None:
                    raise TypeError("a bounded view is not sliced per call")
                return dataclasses.replace(self, shape=(width, *self.shape[1:]),
                                           offset=self._plus(start * row))
            if not (0 <= start <= stop <= n):
                raise IndexError(f"slice {start}:{stop} of {n} rows")
            bound = self.bound
            return dataclasses.replace(self, shape=(stop - start, *self.shape[1:]),
                                       offset=self._plus(start * row), bound=bound)
        if isinstance(index, Expr):
            # one row of a bounded view (the last prompt row, x[rows - 1]) is a plain row
            return dataclasses.replace(self, shape=self.shape[1:], offset=self._plus(index * row), bound=None,
                                       per=Fraction(1))
        i = int(index)
        if i < 0:
            i += n
        if not 0 <= i < n:
            raise IndexError(f"row {index} of {n}")
        return dataclasses.replace(self, shape=self.shape[1:], offset=self._plus(i * row), bound=None,
                                   per=Fraction(1))

    def _plus(self, delta):
        if isinstance(self.offset, Expr) and isinstance(delta, Expr):
            return self.offset + delta
        return self.offset + delta if not isinstance(delta, Expr) else delta + self.offset

    def __setitem__(self, index, value) -> None:
        from ..operators.copy import Copy

        Copy.step(value, self[index] if index is not Ellipsis else self)

    # ---- arithmetic: each records a step ----
    def _binary(self, other, elementwise, rowwise, scalar_fill=None):
        rec = self._rec()
        other = rec.as_handle(other, like=self)
        if tuple(other.shape) == tuple(self.shape):
            y = elementwise.step(self.reshape(self.elements), other.reshape(other.elements))
            return dataclasses.replace(y.reshape(self.shape), bound=self.bound, per=self.per)
        if len(other.shape) == 1 and self.shape and other.shape[0] == self.shape[-1]:
            rows = self.elements // self.shape[-1]
            y = rowwise.step(self.reshape(rows, self.shape[-1]), other)
            return dataclasses.replace(y.reshape(self.shape), bound=self.bound, per=self.per)
        raise ValueError(f"shapes {self.shape} and {other.shape} do not combine")

    def __add__(self, other):
        from ..operators.elementwise_add import ElementwiseAdd, RowwiseAdd

        return self._binary(other, ElementwiseAdd, RowwiseAdd)

    __radd__ = __add__

    def __mul__(self, other):
        from ..operators.elementwise_mul import ElementwiseMul, RowwiseMul

        return self._binary(other, ElementwiseMul, RowwiseMul)

    __rmul__ = __mul__

    def __sub__(self, other):
        from ..operators.axpy import AXPY

        rec = self._rec()
        other = rec.as_handle(other, like=self)
        if tuple(other.shape) != tuple(self.shape):
            raise ValueError(f"shapes {self.shape} and {other.shape} do not subtract")
        y = AXPY.step(other.reshape(other.elements), self.reshape(self.elements), scalar_factor=-1.0)
        return dataclasses.replace(y.reshape(self.shape), bound=self.bound, per=self.per)

    def __truediv__(self, c):
        return self * (1.0 / float(c))

    def __repr__(self):
        return f"Handle({self.buffer.name}{list(self.shape)} +{self.offset}{'' if self.bound is None else f' :{self.bound}'})"
