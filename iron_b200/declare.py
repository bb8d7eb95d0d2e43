"""Operator declaration: fields, operands, construction, recording hook and judging.

The reference splits this between mlir-aie (``param``/``tunable``/``per_call``/``Select``,
``In``/``Out``/``InOut``, the base ``Operator``) and ``iron/common/declare/operator.py:84-725``.
This module restates the host half of both for B200: the same class-body vocabulary, the
same keyword-only construction and error types, ``Cls.step(...)`` recording inside a
graph body, ``op(*tensors)`` standalone dispatch, ``reference/tolerance/ops/judge`` and
``declaration.infer``.  The device half -- ``build()``/``sequence()`` on the NPU -- is one
method here, ``launch(buffers, values)``, which calls the C ABI.  AIE-only tunables
(columns, tile sizes, pipelines) are declared so profiles and model code that pass them
keep working; they are accepted and not used.
"""

from __future__ import annotations

import contextvars
import copy
import itertools
import math
import types
from typing import Any, Callable, Iterable, Mapping

import numpy as np
from ml_dtypes import bfloat16

from .verify import Tolerance, Verdict, compare

MISSING = object()

#: The recorder a ``Graph`` installs while its body runs (iron/common/graph/record.py:542-547).
graph_recorder: contextvars.ContextVar = contextvars.ContextVar("graph_recorder", default=None)


class Unresolvable(Exception):
    """A tunable that no call value, profile or default settles."""


class Field:
    """One declared field of an operator class: a param, a tunable or a per-call value."""

    def __init__(self, kind, default=MISSING, derive=None, domain=None, array=False, repr=True,
                 init=True, bounds=None):
        self.kind, self.default, self.derive, self.domain = kind, default, derive, domain
        self.array, self.repr, self.init, self.bounds = array, repr, init, bounds
        self.name: str = ""

    def __repr__(self):
        return f"<{self.kind} {self.name}>"


def param(default=MISSING, *, derive=None, array=False, repr=True, init=True) -> Any:
    """A construction argument; ``derive`` computes it from other fields instead."""
    return Field("param", default, derive, None, array, repr, init)


def tunable(default=None, *, domain=None, init=True, repr=True) -> Any:
    """A device tunable.  Kept for API parity: accepted at construction, None unless given."""
    return Field("tunable", default, None, domain, False, repr, init)


def per_call(*, derive=None, bounds=None) -> Any:
    """A value that may differ per call.  ``bounds=<param>`` makes it an extent that reads as
    that param until a call (or a graph) binds it lower."""
    return Field("per_call", MISSING, derive, None, False, False, False, bounds)


class Select:
    """``if_true`` where the bool field ``flag`` holds, else ``if_false`` (a dim or a tuple of dims)."""

    def __init__(self, flag, if_true, if_false):
        self.flag, self.if_true, self.if_false = flag, if_true, if_false


class Operand:
    """A declared buffer: direction, dims (fields, ints or ``Select``), dtype, presence flag."""

    def __init__(self, direction: str, dims: tuple, dtype=bfloat16, when=None, like=None, **_aie_only):
        self.direction, self.dims, self.dtype, self.when, self.like = direction, dims, dtype, when, like
        self.name = ""

    def __repr__(self):
        return f"<{self.direction} {self.name}>"


def In(*dims, **kw) -> Any:
    return Operand("in", dims, **kw)


def Out(*dims, **kw) -> Any:
    return Operand("out", dims, **kw)


def InOut(*dims, **kw) -> Any:
    return Operand("inout", dims, **kw)


class Buffer:
    """An operand of one operator instance, its shape resolved."""

    def __init__(self, op: "Operator", decl: Operand):
        self.op, self.decl, self.name = op, decl, decl.name

    @property
    def shape(self) -> tuple[int, ...]:
        return self.op._shape_of(self.decl)

    host_shape = shape

    @property
    def dtype(self):
        d = self.decl.dtype
        return getattr(self.op, d.name) if isinstance(d, Field) else d

    host_dtype = dtype

    @property
    def nbytes(self) -> int:
        return int(np.prod(self.shape, dtype=np.int64)) * np.dtype(self.dtype).itemsize

    @property
    def is_input(self) -> bool:
        return self.decl.direction in ("in", "inout")

    @property
    def is_output(self) -> bool:
        return self.decl.direction in ("out", "inout")

    def __hash__(self):
        return hash((id(self.op), self.name))

    def __eq__(self, other):
        return isinstance(other, Buffer) and other.op is self.op and other.name == self.name

    def __repr__(self):
        return f"{type(self.op).__name__}.{self.name}{self.shape}"


class Declaration:
    """What a class declares, in order."""

    def __init__(self, fields: dict[str, Field], operands: dict[str, Operand]):
        self.members = fields
        self.params = {n: f for n, f in fields.items() if f.kind in ("param", "tunable")}
        self.tunables = {n: f for n, f in fields.items() if f.kind == "tunable"}
        self.per_calls = {n: f for n, f in fields.items() if f.kind == "per_call"}
        self.operands = operands
        # an axis may be absent where its param is None by default or derived (possibly to None)
        self.nullable = {n for n, f in fields.items()
                         if f.kind == "param" and (f.default is None or f.derive is not None)}

    def _flat_dims(self, dims: tuple, flags: Mapping[str, Any]) -> list:
        out = []
        for d in dims:
            if isinstance(d, Select):
                flag = flags.get(d.flag.name, d.flag.default if d.flag.default is not MISSING else False)
                chosen = d.if_true if flag else d.if_false
                out += self._flat_dims(chosen if isinstance(chosen, tuple) else (chosen,), flags)
            else:
                out.append(d)
        return out

    def infer(self, inputs: Mapping[str, tuple[int, ...]], outputs: Mapping[str, tuple[int, ...]] | None = None,
              keep_derived: bool = False, **given) -> dict[str, Any]:
        """Solve construction fields from operand shapes (iron/common/graph/record.py:819-833).

        A dim that is a nullable param may be absent from a shape; the first assignment
        consistent with every shape wins.  Raises ``ValueError`` when none is.
        """
        solved: dict[str, Any] = dict(given)
        shapes = {**inputs, **(outputs or {})}
        for name, shape in shapes.items():
            decl = self.operands[name]
            if decl.when is not None:
                solved.setdefault(decl.when.name, True)
            dims = self._flat_dims(decl.dims, solved)
            optional = [i for i, d in enumerate(dims) if isinstance(d, Field) and d.name in self.nullable]
            drop = len(dims) - len(shape)
            if drop < 0 or drop > len(optional):
                raise ValueError(f"{name}: shape {tuple(shape)} does not fit its {len(dims)} declared axes")
            done = False
            for dropped in itertools.combinations(optional, drop):
                kept = [d for i, d in enumerate(dims) if i not in dropped]
                trial = dict(solved)
                ok = True
                for i in dropped:
                    if trial.setdefault(dims[i].name, None) is not None:
                        ok = False
                for d, extent in zip(kept, shape):
                    if isinstance(d, Field):
                        f = self.members[d.name]
                        if f.derive is not None and f.kind == "param" and not keep_derived:
                            continue  # checked after construction
                        if trial.setdefault(d.name, int(extent)) != int(extent):
                            ok = False
                    elif isinstance(d, int) and d != int(extent):
                        ok = False
                if ok:
                    solved, done = trial, True
                    break
            if not done:
                raise ValueError(f"{name}: shape {tuple(shape)} contradicts the other operands")
        if keep_derived:
            return solved
        return {k: v for k, v in solved.items() if k not in self.members or self.members[k].derive is None}


class OperatorMeta(type):
    def __new__(mcls, name, bases, ns):
        fields: dict[str, Field] = {}
        operands: dict[str, Operand] = {}
        for base in bases:
            decl = getattr(base, "declaration", None)
            if decl is not None:
                fields.update(decl.members)
                operands.update(decl.operands)
        # Operand dims, `when=` flags and `bounds=` name Field objects of this class body,
        # so the objects are named in place rather than copied.
        for key, value in list(ns.items()):
            if isinstance(value, Field):
                value.name = key
                fields[key] = value
                ns.pop(key)
            elif isinstance(value, Operand):
                value.name = key
                operands[key] = value
                ns.pop(key)
        # a dim, `when=` or `like=` may also name its field or operand as a string
        def field_of(d):
            if isinstance(d, str):
                return fields[d]
            if isinstance(d, Select):
                pick = lambda v: tuple(field_of(x) for x in v) if isinstance(v, tuple) else field_of(v)
                return Select(field_of(d.flag), pick(d.if_true), pick(d.if_false))
            return d

        for o in operands.values():
            o.dims = tuple(field_of(d) for d in o.dims)
            if isinstance(o.when, str):
                o.when = fields[o.when]
            if isinstance(o.like, str):
                o.like = operands[o.like]
            if isinstance(o.dtype, str):
                o.dtype = fields[o.dtype]
        for f in fields.values():
            if isinstance(f.bounds, str):
                f.bounds = fields[f.bounds]
        cls = super().__new__(mcls, name, bases, ns)
        cls.declaration = Declaration(fields, operands)
        return cls


class Operator(metaclass=OperatorMeta):
    """Base of every operator.  Subclasses declare fields and operands and implement
    ``reference``, ``tolerance``, ``ops`` and ``launch``."""

    reference_only = False
    declaration: Declaration

    def __init__(self, **kwargs):
        decl = type(self).declaration
        unknown = set(kwargs) - {n for n, f in decl.members.items() if f.kind != "per_call"}
        if unknown:
            raise TypeError(f"{type(self).__name__}() got unexpected {sorted(unknown)}")
        self._values: dict[str, Any] = {}
        self.pinned = {n for n in kwargs if n in decl.tunables}
        self.bound_extents: dict[str, int] = {}
        self.dev = None
        for name, f in decl.members.items():
            if f.kind == "per_call":
                continue
            if name in kwargs:
                self._values[name] = kwargs[name]
            elif f.derive is not None:
                continue
            elif f.default is MISSING:
                raise TypeError(f"{type(self).__name__}() needs {name}")
            else:
                continue
        self.validate()

    # ---- field access ----------------------------------------------------------------
    def __getattr__(self, name):
        # only reached when normal lookup fails: declared fields and operands
        if name.startswith("_") or name in ("pinned", "bound_extents", "dev"):
            raise AttributeError(name)
        decl = type(self).declaration
        f = decl.members.get(name)
        if f is not None:
            if f.kind == "per_call":
                if name in self.bound_extents:
                    return self.bound_extents[name]
                if f.bounds is not None:
                    return getattr(self, f.bounds.name)
                if f.derive is not None:
                    return f.derive(self)
                raise AttributeError(name)
            if name in self._values:
                return self._values[name]
            if f.derive is not None:
                return f.derive(self)
            return f.default(self) if isinstance(f.default, types.FunctionType) and f.kind == "param" else f.default
        o = decl.operands.get(name)
        if o is not None:
            return Buffer(self, o)
        raise AttributeError(f"{type(self).__name__} has no {name}")

    def _shape_of(self, decl: Operand) -> tuple[int, ...]:
        if decl.like is not None:
            return self._shape_of(type(self).declaration.operands[decl.like.name])
        flags = {n: getattr(self, n) for n in type(self).declaration.params}
        out = []
        for d in type(self).declaration._flat_dims(decl.dims, flags):
            v = getattr(self, d.name) if isinstance(d, Field) else d
            if v is not None:
                out.append(int(v))
        return tuple(out)

    def _present(self, decl: Operand) -> bool:
        return decl.when is None or bool(getattr(self, decl.when.name))

    @property
    def buffers(self) -> list[Buffer]:
        """Inputs then outputs, the order a standalone call takes its tensors in."""
        return self.inputs + [b for b in self.outputs if b.decl.direction == "out"]

    @property
    def inputs(self) -> list[Buffer]:
        d = type(self).declaration
        return [Buffer(self, o) for o in d.operands.values() if o.direction in ("in", "inout") and self._present(o)]

    @property
    def outputs(self) -> list[Buffer]:
        d = type(self).declaration
        return [Buffer(self, o) for o in d.operands.values() if o.direction in ("out", "inout") and self._present(o)]

    def replace(self, **changes) -> "Operator":
        new = copy.copy(self)
        new._values = {**self._values, **changes}
        new.bound_extents = dict(self.bound_extents)
        return new

    def bind(self, **extents: int) -> "Operator":
        """This operator with per-call extents bound (a bounded call's view of it)."""
        decl = type(self).declaration
        for name, v in extents.items():
            f = decl.per_calls.get(name)
            if f is None:
                raise TypeError(f"{type(self).__name__} has no per-call value {name}")
            if f.bounds is not None and not 0 <= int(v) <= getattr(self, f.bounds.name):
                raise IndexError(f"{name}={v} is outside 0..{getattr(self, f.bounds.name)}")
        new = copy.copy(self)
        new.bound_extents = {**self.bound_extents, **{k: int(v) for k, v in extents.items()}}
        return new

    def __repr__(self):
        decl = type(self).declaration
        shown = ", ".join(f"{n}={self._values[n]!r}" for n, f in decl.members.items()
                          if n in self._values and f.repr)
        return f"{type(self).__name__}({shown})"

    @property
    def name(self) -> str:
        return type(self).__name__

    # ---- hooks a subclass may define -------------------------------------------------
    def validate(self) -> None:
        """Raise ``ValueError`` for a shape the operator refuses (at construction)."""

    def resolved(self, dev=None) -> "Operator":
        """The operator with its tunables settled.  Nothing on B200 depends on them."""
        return self

    def reference(self, *inputs, **values):
        raise NotImplementedError

    def tolerance(self) -> Tolerance | None:
        raise NotImplementedError

    def ops(self) -> int:
        raise NotImplementedError

    def launch(self, buffers: dict, values: dict) -> None:
        """Run on the device: ``buffers`` maps operand names to CUDA tensors; ``values`` maps
        per-call names to ints or to one-element int32 device tensors."""
        raise NotImplementedError

    # ---- recording and dispatch --------------------------------------------------------
    @classmethod
    def step(cls, *operands, **kwargs):
        """Record one step of this operator in the graph body being run."""
        rec = graph_recorder.get()
        if rec is None:
            raise TypeError(f"{cls.__name__}.step() records a step in a Graph's body; "
                            f"construct the operator and call it to run it alone")
        return rec.call(cls, operands, kwargs)

    @classmethod
    def call_operands(cls, operands: tuple, kwargs: dict) -> tuple[dict, dict, dict]:
        """Split a ``step`` call into inputs by name, given outputs by name and field kwargs
        (iron/common/declare/operator.py:241-260): positional operands are the inputs in
        declaration order, then outputs; an optional input comes by keyword."""
        decl = cls.declaration
        ins = [o for o in decl.operands.values() if o.direction in ("in", "inout")]
        outs = [o for o in decl.operands.values() if o.direction == "out"]
        required = [o for o in ins if o.when is None]
        if len(operands) > len(required) + len(outs):
            raise TypeError(f"{cls.__name__} takes at most {len(required) + len(outs)} operands")
        given_in = {o.name: v for o, v in zip(required, operands)}
        given_out = {o.name: v for o, v in zip(outs, operands[len(required):])}
        fields = {}
        for k, v in kwargs.items():
            o = decl.operands.get(k)
            if o is not None:
                if v is None:
                    continue
                (given_in if o.direction != "out" else given_out)[k] = v
            else:
                fields[k] = v
        if len(given_in) < len(required) and len(operands) < len(required):
            missing = [o.name for o in required if o.name not in given_in]
            raise TypeError(f"{cls.__name__} is missing operands {missing}")
        for name in given_in:
            o = decl.operands[name]
            if o.when is not None:
                if fields.get(o.when.name, True) is False:
                    raise TypeError(f"{cls.__name__}: {name} given but {o.when.name} is False")
                fields[o.when.name] = True
        return given_in, given_out, fields

    def __call__(self, *tensors, **values):
        rec = graph_recorder.get()
        if rec is not None:
            return rec.call(type(self), tensors, {**self._values, **values})
        from .tensor import as_device

        bufs = self.buffers
        if len(tensors) != len(bufs):
            raise TypeError(f"{self.name} takes {len(bufs)} tensors ({[b.name for b in bufs]}), got {len(tensors)}")
        device = {}
        for b, t in zip(bufs, tensors):
            dt = as_device(t)
            if tuple(dt.shape) != b.shape:
                raise ValueError(f"{self.name}.{b.name} is {b.shape}, got {tuple(dt.shape)}")
            device[b.name] = dt.torch
        self.bind(**values).launch(device, dict(values))
        return tensors[len(self.inputs):] if len(bufs) - len(self.inputs) != 1 else tensors[-1]

    # ---- judging -----------------------------------------------------------------------
    def _call_reference(self, inputs: Mapping[str, np.ndarray], **values) -> dict[str, np.ndarray]:
        op = self.bind(**values) if values else self
        out = op.reference(*[inputs[b.name] for b in op.inputs])
        outs = [b for b in op.outputs]
        if not isinstance(out, tuple):
            out = (out,)
        return {b.name: np.asarray(o) for b, o in zip(outs, out)}

    def judge(self, inputs: Mapping[str, np.ndarray], written: Mapping[str, np.ndarray],
              tolerance: Tolerance | None = None, expected: Mapping[str, np.ndarray] | None = None,
              **values) -> dict[str, Verdict]:
        """Compare each written output with the reference's under ``tolerance`` (the operator's own)."""
        tol = self.tolerance() if tolerance is None else tolerance
        if tol is None:
            raise TypeError(f"{self.name} states no tolerance")
        want = self._call_reference(inputs, **values) if expected is None else expected
        bound = None
        if tol.kind == "bound":
            bound = tol.bound(*[inputs[b.name] for b in self.inputs])
        return {name: compare(written[name], want[name], tol, bound=bound) for name in written}


def ceildiv(a: int, b: int) -> int:
    return -(-a // b)


def __getattr__(name):
    # ``Profile`` lives beside the declarations (iron/common/declare/__init__.py exports both)
    if name == "Profile":
        from .profile import Profile

        return Profile
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
