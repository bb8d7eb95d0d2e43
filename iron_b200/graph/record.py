"""Recording a graph's body into steps, and running a recording on the host.

``Recorder`` is what ``Operator.step`` talks to while a body runs
(iron/common/graph/record.py:480-1010): it turns arrays, params and states into handles,
solves each operator's fields from its operands' shapes, binds per-call bounds and
offsets, and allocates the outputs.  ``Recording.reference`` replays the steps with every
operator's numpy ``reference()`` over byte-exact host buffers, writing only the bounded
rows, with states persisting between calls (record.py:340-448) -- the device-free model
path the parity tests use.
"""

from __future__ import annotations

import dataclasses
import math
from typing import Any, Mapping

import numpy as np

from ..declare import Field, Operator, graph_recorder
from .expr import Expr, evaluate
from .handle import BufferRef, Handle, Held, Param, State, Weight


@dataclasses.dataclass
class Step:
    op: Operator
    inputs: dict[str, Handle]
    outputs: dict[str, Handle]
    values: dict[str, Any]          # per-call name -> int or Expr
    index: int = 0

    @property
    def name(self) -> str:
        return f"{self.index}:{self.op.name}"


@dataclasses.dataclass
class Carry:
    """What a call carries to the next: names to per-call expressions or one-element handles."""

    values: dict[str, Any]


def carry(**values) -> Carry:
    return Carry(values)


class Recorder:
    def __init__(self, graph_name: str = "graph", profile=None):
        self.graph_name = graph_name
        self.profile = profile      # a Profile: fills the tunables a step's construction leaves open
        self.steps: list[Step] = []
        self.buffers: list[BufferRef] = []
        self._held: dict[int, BufferRef] = {}
        self._consts: dict[tuple, BufferRef] = {}
        self._token = None
        # (first row, rows moved, rows of the buffer, what): first + moved <= buffer, checked per call;
        # a run bounded per call moves only its bound's rows, so only those must lie inside
        self.limits: list[tuple[Any, Any, int, str]] = []

    # ---- context ----
    def __enter__(self):
        self._token = graph_recorder.set(self)
        return self

    def __exit__(self, *exc):
        graph_recorder.reset(self._token)

    # ---- buffers and handles ----
    def _new(self, kind, name, shape, dtype, held=None) -> BufferRef:
        buf = BufferRef(kind, f"{name}#{len(self.buffers)}", tuple(int(s) for s in shape), dtype, held)
        self.buffers.append(buf)
        return buf

    def input(self, name: str, shape, dtype) -> Handle:
        buf = self._new("input", name, shape, dtype)
        return Handle(buf, buf.shape)

    def transient(self, name: str, shape, dtype) -> Handle:
        buf = self._new("transient", name, shape, dtype)
        return Handle(buf, buf.shape)

    def handle_of(self, held: Held) -> Handle:
        buf = self._held.get(id(held))
        if buf is None:
            if isinstance(held, Param) and held.array is None:
                raise TypeError(f"{self.graph_name}: a param of shape {held.shape} was never loaded")
            kind = "state" if isinstance(held, State) else "weight"
            buf = self._new(kind, type(held).__name__.lower(), held.shape, held.dtype, held)
            self._held[id(held)] = buf
        return Handle(buf, buf.shape)

    def as_handle(self, x, like: Handle | None = None) -> Handle:
        if isinstance(x, Handle):
            return x
        if isinstance(x, Held):
            return self.handle_of(x)
        if isinstance(x, np.ndarray):
            w = Weight(x)
            self._keep = getattr(self, "_keep", []) + [w]
            return self.handle_of(w)
        if isinstance(x, (int, float)) and like is not None:
            # a scalar becomes a constant row of the view's last axis
            key = (float(x), like.shape[-1], np.dtype(like.dtype).name)
            buf = self._consts.get(key)
            if buf is None:
                w = Weight(np.full((like.shape[-1],), x, dtype=like.dtype))
                self._keep = getattr(self, "_keep", []) + [w]
                buf = self.handle_of(w).buffer
                self._consts[key] = buf
            return Handle(buf, buf.shape)
        raise TypeError(f"{type(x).__name__} is not an operand")

    # ---- recording a step ----
    def call(self, cls: type, operands: tuple, kwargs: dict):
        from ..operators.copy import Copy, Gather

        if cls is Copy:
            return self._copy(operands, kwargs)
        given_in, given_out, fields = cls.call_operands(operands, kwargs)
        ins = {n: self._materialise(self.as_handle(v)) for n, v in given_in.items()}
        outs = {n: self.as_handle(v) for n, v in given_out.items()}
        # An output given as a view at a per-call offset (a state's slot picked by the call's
        # position) is computed into a transient and copied there: only Copy resolves a
        # per-call offset on the device.
        placed_later = []
        for n, h in list(outs.items()):
            if isinstance(h.offset, Expr):
                tmp = self.transient(f"{cls.__name__}.{n}", h.shape, h.dtype)
                placed_later.append((tmp, h))
                outs[n] = tmp
        decl = cls.declaration
        per_call_given = {k: fields.pop(k) for k in list(fields) if k in decl.per_calls}
        shapes = {n: h.shape for n, h in ins.items()}
        solved = decl.infer(shapes, {n: h.shape for n, h in outs.items()}, keep_derived=True,
                            **{k: v for k, v in fields.items() if v is not None or k in decl.nullable})
        adopt = getattr(cls, "adopt", None)
        if adopt is not None:
            solved = adopt(solved)   # a class may read a derived axis to fill a field it defaults from
        solved = {k: v for k, v in solved.items() if k not in decl.members or decl.members[k].derive is None}
        op = cls(**solved) if self.profile is None else self.profile.make(cls, **solved)
        values: dict[str, Any] = dict(per_call_given)
        # a bound on an operand's leading axis binds the extent that axis sizes
        for name, h in ins.items():
            if h.bound is None:
                continue
            extent = self._extent_for(op, decl.operands[name])
            if extent is None:
                raise TypeError(f"{cls.__name__}.{name}: its leading axis cannot be bounded per call")
            values[extent] = h.rows_bound()
        out_handles = {}
        for b in op.outputs:
            if b.decl.direction == "inout":
                out_handles[b.name] = ins[b.name]
                continue
            h = outs.get(b.name) or self.transient(f"{cls.__name__}.{b.name}", b.shape, b.dtype)
            if tuple(h.shape) != b.shape:
                raise ValueError(f"{cls.__name__}.{b.name} is {b.shape}, given {h.shape}")
            # the output's leading rows are bounded as the input sizing the same axis is
            extent = self._extent_for(op, b.decl)
            if extent in values and h.bound is None:
                h = dataclasses.replace(h, bound=values[extent])
            out_handles[b.name] = h
        step = Step(op, ins, out_handles, values, len(self.steps))
        self.steps.append(step)
        for tmp, view in placed_later:
            self._copy((tmp, view), {})
        results = [out_handles[b.name] for b in op.outputs]
        return results[0] if len(results) == 1 else tuple(results)

    @staticmethod
    def _extent_for(op: Operator, operand) -> str | None:
        decl = type(op).declaration
        dims = decl._flat_dims(operand.dims, {n: getattr(op, n) for n in decl.params})
        lead = next((d for d in dims if not (isinstance(d, Field) and getattr(op, d.name) is None)), None)
        if not isinstance(lead, Field):
            return None
        for name, f in decl.per_calls.items():
            if f.bounds is lead:
                return name
        return None

    def _materialise(self, h: Handle) -> Handle:
        """A view an operator can read in place, or a copy of one it cannot (a gather, or a
        per-call offset, which only Copy resolves on the device)."""
        if h.ids is not None or isinstance(h.offset, Expr):
            return self._copy((h,), {})
        return h

    def _copy(self, operands: tuple, kwargs: dict) -> Handle:
        from ..operators.copy import Copy, Gather

        kwargs = {k: v for k, v in kwargs.items() if k != "dtype"}
        src = self.as_handle(operands[0])
        dst = self.as_handle(operands[1]) if len(operands) > 1 else None
        if src.ids is not None:
            ids, table = src.ids, dataclasses.replace(src, ids=None, shape=src.buffer.shape, bound=None)
            if isinstance(table.offset, Expr) or table.offset != 0 or len(table.shape) != 2:
                raise TypeError("rows are gathered from a whole two-dimensional table")
            op = Gather(rows=ids.shape[0], cols=table.shape[1], table_rows=table.shape[0])
            out = dst or self.transient("Gather.out", (ids.shape[0], table.shape[1]), table.dtype)
            values = {}
            if ids.bound is not None:
                values["valid"] = ids.rows_bound()
                out = dataclasses.replace(out, bound=ids.bound, per=ids.per)
            step = Step(op, {"table": table, "ids": self._materialise(ids)}, {"out": out}, values, len(self.steps))
            self.steps.append(step)
            return out
        shape = src.shape
        if dst is not None and math.prod(dst.shape) != math.prod(shape):
            raise ValueError(f"copy of {shape} into {dst.shape}")
        rows = shape[0] if len(shape) > 1 else 1
        cols = int(math.prod(shape)) // rows
        if dst is None:
            dst = self.transient("Copy.dst", shape, src.dtype)
            if src.bound is not None:
                dst = dataclasses.replace(dst, bound=src.bound, per=src.per)
        values: dict[str, Any] = {}
        bound = src.bound if src.bound is not None else dst.bound
        bound_h = src if src.bound is not None else dst
        if bound is not None:
            values["valid"] = bound_h.rows_bound() if len(shape) > 1 else 1
        for name, h in (("src_row", src), ("dst_row", dst)):
            off = h.offset
            if isinstance(off, Expr):
                scaled = self._rows_of(off, cols)
                values[name] = scaled
                total = h.buffer.elements // cols
                self.limits.append((scaled, values.get("valid", rows), total, f"{h.buffer.name} rows"))
            else:
                if off % cols:
                    raise TypeError("a copied view starts on a row boundary")
                values[name] = off // cols
        op = Copy(rows=rows, cols=cols, src_rows=src.buffer.elements // cols,
                  dst_rows=dst.buffer.elements // cols, dtype=src.dtype)
        if np.dtype(src.dtype) != np.dtype(dst.dtype):
            raise TypeError("a copy keeps the element type")
        whole = lambda h: Handle(h.buffer, (h.buffer.elements // cols, cols))
        step = Step(op, {"src": whole(src)}, {"dst": whole(dst)}, values, len(self.steps))
        self.steps.append(step)
        return dst

    @staticmethod
    def _rows_of(offset: Expr, cols: int) -> Expr:
        """An element offset as a row offset: every term must be a multiple of ``cols``."""
        if offset.mul % cols or offset.add % cols:
            if offset.linear:
                f = offset._flat()
                if f.scale % cols == 0 and f.bias % cols == 0:
                    return Expr(f.name, f.scale // cols, f.bias // cols)
            raise TypeError("a copied view starts on a row boundary")
        return dataclasses.replace(offset, mul=offset.mul // cols, add=offset.add // cols)


class Recording:
    """The steps one call signature records, and what the body returned."""

    def __init__(self, recorder: Recorder, inputs: dict[str, Handle], outputs, carried: Carry | None,
                 value_names: list[str]):
        self.steps, self.buffers = recorder.steps, recorder.buffers
        self.inputs, self.outputs, self.carried = inputs, outputs, carried
        self.value_names, self.limits = value_names, recorder.limits
        self._recorder = recorder  # keeps the constants it made alive

    def check_limits(self, values: Mapping[str, int]) -> None:
        """Refuse a call whose per-call indices or bounds leave their buffers, before any dispatch."""
        for first, moved, total, what in self.limits:
            v, n = evaluate(first, values), evaluate(moved, values)
            if v < 0 or n < 0 or v + n > total:
                raise IndexError(f"{what}: rows {v}..{v + n} are outside 0..{total} for {dict(values)}")
        for step in self.steps:
            for name, e in step.values.items():
                f = type(step.op).declaration.per_calls.get(name)
                if f is not None and f.bounds is not None:
                    v = evaluate(e, values)
                    top = getattr(step.op, f.bounds.name)
                    if not 0 <= v <= top:
                        raise IndexError(f"{step.name}: {name}={v} is outside 0..{top}")

    def reference(self, arrays: Mapping[str, np.ndarray], values: Mapping[str, int]):
        """Run every step's ``reference()`` on the host; returns ``(outputs, carried)``."""
        self.check_limits(values)
        store: dict[int, np.ndarray] = {}

        def backing(buf: BufferRef) -> np.ndarray:
            arr = store.get(id(buf))
            if arr is None:
                if buf.kind == "input":
                    arr = np.ascontiguousarray(arrays[buf.name.split("#")[0]]).reshape(-1).astype(buf.dtype)
                elif buf.kind == "weight":
                    arr = np.asarray(buf.held.array).reshape(-1)
                elif buf.kind == "state":
                    if buf.held.host is None:
                        buf.held.host = np.zeros(buf.elements, buf.dtype)
                    arr = buf.held.host
                else:
                    arr = np.zeros(buf.elements, buf.dtype)
                store[id(buf)] = arr
            return arr

        def read(h: Handle) -> np.ndarray:
            off = evaluate(h.offset, values)
            return backing(h.buffer)[off : off + h.elements].reshape(h.shape)

        for step in self.steps:
            bound = {n: evaluate(e, values) for n, e in step.values.items()}
            op = step.op.bind(**bound) if bound else step.op
            ins = [read(step.inputs[b.name]) for b in op.inputs]
            out = op.reference(*ins)
            out = out if isinstance(out, tuple) else (out,)
            for b, o in zip(op.outputs, out):
                h = step.outputs[b.name]
                view = read(h)
                o = np.asarray(o).reshape(h.shape)
                rows = None if h.bound is None else evaluate(h.rows_bound(), values)
                if type(op).__name__ == "Copy":
                    r0, n = bound.get("dst_row", 0), bound.get("valid", op.rows)
                    view[r0 : r0 + n] = o[r0 : r0 + n]
                elif rows is None or not h.shape:
                    view[...] = o
                else:
                    view[:rows] = o[:rows]
        outs = self.outputs
        result = tuple(np.array(read(h)) for h in outs) if isinstance(outs, tuple) else (
            None if outs is None else np.array(read(outs)))
        carried = None
        if self.carried is not None:
            carried = {}
            for name, v in self.carried.values.items():
                carried[name] = int(read(v).reshape(-1)[0]) if isinstance(v, Handle) else evaluate(v, values)
        return result, carried
