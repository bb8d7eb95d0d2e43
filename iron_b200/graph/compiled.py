"""``Graph``: a body recorded once per input signature, compiled to one CUDA graph.

The contract of ``iron/common/graph/compiled.py`` (``Graph`` :236-742, ``CompiledGraph``
:745-1051): ``body``'s positional parameters are the inputs, its keyword-only ones the
per-call integer values; weights and states are what the instance holds, by attribute
path; ``compile(**shapes)`` records the body on handles and returns a callable version;
a new shape is a new compile; ``reference(...)`` runs the same recording on the host.

On B200 "compile" means: place every buffer of the recording in the graph's device arena
(residents keep one offset in every version, transients share bytes by live range),
upload the weights once, resolve every step to a launch closure over arena slices, and
capture the whole step list as one CUDA graph.  A call copies the inputs and one small
int32 vector of per-call values to the device and replays the graph; per-call bounds and
offsets are read by the kernels from that vector, so intermediates never leave HBM and a
replay launches nothing from the host but the graph.
"""

from __future__ import annotations

import inspect
import math
from typing import Any, Mapping

import numpy as np

from ..arena import ArenaPlan
from ..declare import Operator
from .expr import Expr, evaluate
from .handle import BufferRef, Handle, Held, Param, State, Weight
from .record import Carry, Recorder, Recording, Step


class _Marker:
    """``Scratchpad[np.int32]`` / ``Carried[np.int32]`` annotate a body's per-call values."""

    def __init__(self, kind):
        self.kind = kind

    def __getitem__(self, dtype):
        return (self.kind, dtype)


Scratchpad = _Marker("scratchpad")
Carried = _Marker("carried")


def walk(node, path: str = "", seen=None):
    """Yield ``(path, value, owner, attribute)`` for everything a graph holds, depth first."""
    seen = set() if seen is None else seen
    if id(node) in seen:
        return
    seen.add(id(node))
    items = []
    if isinstance(node, Graph):
        items = [(k, v) for k, v in vars(node).items() if not k.startswith("_")]
    elif isinstance(node, (list, tuple)):
        items = [(str(i), v) for i, v in enumerate(node)]
    elif isinstance(node, dict):
        items = [(str(k), v) for k, v in node.items()]
    for key, value in items:
        sub = f"{path}.{key}" if path else key
        if isinstance(value, (Held, np.ndarray)):
            yield sub, value, node, key
        elif isinstance(value, (Graph, list, tuple, dict)):
            yield from walk(value, sub, seen)


class StepCheckFailed(AssertionError):
    """A step of a graph compiled with ``check=True`` wrote something outside its tolerance."""


class MissingWeights(KeyError):
    """``load_state_dict`` found no array for some of a graph's params."""

    def __init__(self, graph: str, names: list[str]):
        self.names = list(names)
        super().__init__(f"{graph}: the weights lack {self.names}")


class Graph:
    """Subclass it, define ``body``; see the module docstring."""

    profile = None

    def body(self, *inputs, **values):
        raise NotImplementedError(f"{type(self).__name__} defines no body()")

    # ---- calling a graph inside another graph's body records there ----
    def __call__(self, *args, **kwargs):
        from ..declare import graph_recorder

        if graph_recorder.get() is None:
            raise TypeError(f"{type(self).__name__} is called inside a Graph's body; compile() it to run it")
        return self.body(*args, **kwargs)

    @property
    def name(self) -> str:
        return type(self).__name__

    # ---- weights ----
    def load_state_dict(self, tree: Mapping[str, np.ndarray], *, path: str = "") -> None:
        """Bind every ``param`` this graph holds to ``tree``'s array at its attribute path.

        Module by module, as ``torch.nn.Module`` loads: a held graph loads its own attributes
        through its own ``load_state_dict`` (``path`` its dotted prefix), so a subclass can
        override it to derive what it computes with from what it just loaded
        (iron/common/graph/compiled.py:430-470; iron/lm/causal.py:153-157 builds a
        convolution's tap rows this way)."""
        missing: list[str] = []
        self._load_into(self, tree, path, missing, set())
        if missing:
            raise MissingWeights(self.name, missing)

    @staticmethod
    def _load_into(node, tree, path, missing, seen) -> None:
        if isinstance(node, Graph):
            items = [(k, v) for k, v in vars(node).items() if not k.startswith("_")]
        elif isinstance(node, (list, tuple)):
            items = [(str(i), v) for i, v in enumerate(node)]
        elif isinstance(node, dict):
            items = [(str(k), v) for k, v in node.items()]
        else:
            return
        for key, value in items:
            full = f"{path}.{key}" if path else key
            if isinstance(value, Param):
                if full in tree:
                    arr = np.ascontiguousarray(tree[full])
                    if tuple(arr.shape) != tuple(value.shape):
                        raise ValueError(f"{full} is {arr.shape}, the graph holds {value.shape}")
                    value.array, value.dtype = arr, arr.dtype
                elif value.array is None:
                    missing.append(full)
            elif isinstance(value, Graph):
                if id(value) in seen:
                    continue
                seen.add(id(value))
                try:
                    value.load_state_dict(tree, path=full)
                except MissingWeights as e:   # one report for everything every module lacks
                    missing.extend(e.names)
            elif isinstance(value, (list, tuple, dict)):
                Graph._load_into(value, tree, full, missing, seen)

    # ---- recording ----
    def resolved_profile(self):
        """The ``Profile`` this graph's steps are made through (iron/common/graph/compiled.py:734-742):
        ``profile`` may be one, a JSON file, or a directory holding one file per device
        (``b200.json`` is the one read here); None where there is none."""
        from pathlib import Path

        from ..profile import Profile

        held = self.__dict__.get("_profile_loaded")
        if held is not None:
            return held[0]
        given = self.profile
        loaded = None
        if isinstance(given, Profile):
            loaded = given
        elif given is not None:
            path = Path(given)
            if path.is_dir():
                path = path / "b200.json"
            if path.exists():
                loaded = Profile.load(path)
        self.__dict__["_profile_loaded"] = (loaded,)
        return loaded

    def _parameters(self):
        sig = inspect.signature(type(self).body)
        params = list(sig.parameters.values())[1:]
        inputs = [p for p in params if p.kind in (p.POSITIONAL_ONLY, p.POSITIONAL_OR_KEYWORD)]
        values = [p for p in params if p.kind == p.KEYWORD_ONLY]
        return inputs, values

    def record(self, **shapes) -> Recording:
        """Run ``body`` on handles for inputs of ``shapes`` (``name=(shape, dtype)``)."""
        inputs, values = self._parameters()
        rec = Recorder(self.name, self.resolved_profile())
        handles, names = [], []
        for p in inputs:
            if p.name in shapes:
                shape, dtype = shapes[p.name]
                handles.append(rec.input(p.name, shape, dtype))
                names.append(p.name)
            elif p.default is None:
                handles.append(None)
            else:
                raise TypeError(f"{self.name}.compile() needs the shape of input {p.name}")
        unknown = set(shapes) - {p.name for p in inputs}
        if unknown:
            raise TypeError(f"{self.name} has no input {sorted(unknown)}")
        exprs = {p.name: Expr(p.name) for p in values}
        with rec:
            out = self.body(*handles, **exprs)
        carried = None
        if isinstance(out, tuple) and out and isinstance(out[-1], Carry):
            carried, out = out[-1], out[:-1]
            out = out[0] if len(out) == 1 else out
        elif isinstance(out, Carry):
            carried, out = out, None
        return Recording(rec, {n: h for n, h in zip(names, [h for h in handles if h is not None])}, out, carried,
                         [p.name for p in values])

    @staticmethod
    def _signature(shapes) -> tuple:
        return tuple((n, tuple(s), np.dtype(d).name) for n, (s, d) in shapes.items())

    def compile(self, *, check: bool = False, **shapes) -> "CompiledGraph":
        """The version for inputs of ``shapes``; compiled once per signature.

        ``check=True`` gives a version that runs every step as a launch of its own and holds
        what it wrote to the step's ``reference()`` on the very inputs the device read, inside
        the step's ``tolerance()``, raising ``StepCheckFailed`` at the first step outside it
        (iron/common/graph/compiled.py:556-557, iron/common/image/callable.py:785-797): the
        way to find which kernel of a graph is wrong."""
        versions = self.__dict__.setdefault("_versions", {})
        key = (self._signature(shapes), bool(check))
        if key not in versions:
            plan = self.__dict__.setdefault("_plan", ArenaPlan())
            versions[key] = CompiledGraph(self, self.record(**shapes), plan, check=check)
        return versions[key]

    def reference(self, *arrays, **values):
        """Run the body's recording on the host with every step's ``reference()``."""
        inputs, value_params = self._parameters()
        shapes = {p.name: (np.asarray(a).shape, np.asarray(a).dtype) for p, a in zip(inputs, arrays) if a is not None}
        refs = self.__dict__.setdefault("_references", {})
        key = self._signature(shapes)
        if key not in refs:
            refs[key] = self.record(**shapes)
        rec = refs[key]
        vals = _check_values(self.name, value_params, values)
        out, carried = rec.reference({n: np.asarray(a) for n, a in zip(rec.inputs, [a for a in arrays if a is not None])}, vals)
        return out if carried is None else (out, carried) if out is not None else carried


def _check_values(name, params, given: Mapping[str, Any]) -> dict[str, int]:
    unknown = set(given) - {p.name for p in params}
    if unknown:
        raise TypeError(f"{name} takes no per-call value {sorted(unknown)}")
    out = {}
    for p in params:
        if p.name in given:
            v = given[p.name]
        elif p.default is not inspect.Parameter.empty:
            v = p.default
        else:
            raise TypeError(f"{name} needs the per-call value {p.name}")
        if isinstance(v, (bool, float)) or not isinstance(v, (int, np.integer)):
            raise TypeError(f"{name}: per-call value {p.name} must be an integer, got {type(v).__name__}")
        out[p.name] = int(v)
    return out


class DeviceBuffer:
    """A buffer of a compiled graph as the caller sees it."""

    def __init__(self, tensor):
        self.torch = tensor

    def numpy(self) -> np.ndarray:
        from ..tensor import torch_to_numpy

        return torch_to_numpy(self.torch)

    @property
    def shape(self):
        return tuple(self.torch.shape)


_TORCH = {"bfloat16": "bfloat16", "float32": "float32", "int32": "int32", "float16": "float16", "int64": "int64"}


class CompiledGraph:
    """One version of a graph on the device."""

    def __init__(self, graph: Graph, recording: Recording, plan: ArenaPlan, check: bool = False):
        import torch

        self.check = check

        if not torch.cuda.is_available():
            raise RuntimeError("compile() needs a CUDA device; Graph.reference() runs on the host")
        for step in recording.steps:
            if step.op.reference_only:
                raise TypeError(f"{step.name} is reference-only and cannot be compiled")
        self.graph, self.recording = graph, recording
        self._torch = torch
        self.device = torch.device("cuda")
        # ---- place every buffer ----
        sizes = {b.name: max(b.nbytes, 16) for b in recording.buffers}
        residents = {b.name: id(b.held) for b in recording.buffers if b.kind in ("weight", "state")}
        touched = []
        io = [h.buffer.name for h in recording.inputs.values()]
        outs = recording.outputs if isinstance(recording.outputs, tuple) else (
            () if recording.outputs is None else (recording.outputs,))
        io += [h.buffer.name for h in outs]
        touched.append(list(io))   # inputs and outputs live for the whole call
        for step in recording.steps:
            touched.append([h.buffer.name for h in (*step.inputs.values(), *step.outputs.values())])
        touched.append(list(io))
        self.spans = plan.place_version(touched, sizes, residents)
        store = graph.__dict__.setdefault("_storage", {})
        arena = store.get("arena")
        if arena is None or arena.numel() < plan.size:
            new = torch.zeros(plan.size, dtype=torch.uint8, device=self.device)
            if arena is not None:
                new[: arena.numel()].copy_(arena)   # residents keep their offsets and contents
            store["arena"] = arena = new
            for other in graph.__dict__.get("_versions", {}).values():
                other._bind(arena)
        self._uploaded = store.setdefault("uploaded", set())
        self._bind(arena)
        # ---- per-call values: one int32 slot per distinct expression ----
        self._slots: dict[Expr, int] = {}
        for step in recording.steps:
            for e in step.values.values():
                if isinstance(e, Expr):
                    self._slots.setdefault(e, len(self._slots))
        n = max(len(self._slots), 1)
        self._values = torch.zeros(n, dtype=torch.int32, device=self.device)
        self._ring = [torch.zeros(n, dtype=torch.int32).pin_memory() for _ in range(8)]
        self._ring_done = [None] * 8
        self._ring_at = 0
        self._cuda_graph = None

    def _bind(self, arena) -> None:
        torch = self._torch
        self.arena = arena
        self.tensors: dict[str, Any] = {}
        for b in self.recording.buffers:
            s = self.spans[b.name]
            dt = getattr(torch, _TORCH[np.dtype(b.dtype).name])
            self.tensors[b.name] = arena[s.offset : s.offset + b.nbytes].view(dt)
        self._cuda_graph = None
        self.upload()

    def upload(self) -> None:
        """Copy every weight not yet on the device into its arena slice (once per graph)."""
        from ..tensor import numpy_to_torch

        for b in self.recording.buffers:
            if b.kind == "weight" and id(b.held) not in self._uploaded:
                self.tensors[b.name].copy_(numpy_to_torch(np.asarray(b.held.array).reshape(-1), self.device))
                self._uploaded.add(id(b.held))

    # ---- running ----
    def _view(self, h: Handle):
        off = h.offset if isinstance(h.offset, int) else 0
        return self.tensors[h.buffer.name][off : off + h.elements].view(*h.shape) if h.shape else \
            self.tensors[h.buffer.name][off : off + 1]

    def _launch_all(self) -> None:
        for step in self.recording.steps:
            static = {n: v for n, v in step.values.items() if not isinstance(v, Expr)}
            op = step.op.bind(**static) if static else step.op
            vals = {f"d_{n}": self._values[self._slots[v] : self._slots[v] + 1]
                    for n, v in step.values.items() if isinstance(v, Expr)}
            bufs = {n: self._view(h) for n, h in (*step.inputs.items(), *step.outputs.items())}
            op.launch(bufs, vals)

    def _launch_checked(self, vals: Mapping[str, int]) -> None:
        """Every step alone: read its inputs back, launch it, read what it wrote, and judge that
        against the step's numpy reference on those inputs (only the rows the call bounds)."""
        from ..tensor import torch_to_numpy
        from ..verify import compare

        torch = self._torch
        for step in self.recording.steps:
            bound = {n: evaluate(e, vals) for n, e in step.values.items()}
            op = step.op.bind(**bound) if bound else step.op
            tol = op.tolerance()
            if tol is None:
                raise StepCheckFailed(f"{step.name} states no tolerance to be held to")
            torch.cuda.synchronize()
            ins = {b.name: torch_to_numpy(self._view(step.inputs[b.name])).copy() for b in op.inputs}
            before = {b.name: torch_to_numpy(self._view(step.outputs[b.name])).copy() for b in op.outputs}
            static = {n: v for n, v in step.values.items() if not isinstance(v, Expr)}
            launch_op = step.op.bind(**static) if static else step.op
            dvals = {f"d_{n}": self._values[self._slots[v] : self._slots[v] + 1]
                     for n, v in step.values.items() if isinstance(v, Expr)}
            bufs = {n: self._view(h) for n, h in (*step.inputs.items(), *step.outputs.items())}
            launch_op.launch(bufs, dvals)
            torch.cuda.synchronize()
            out = op.reference(*[ins[b.name] for b in op.inputs])
            out = out if isinstance(out, tuple) else (out,)
            bound_fn = tol.bound(*[ins[b.name] for b in op.inputs]) if tol.kind == "bound" else None
            for b, want in zip(op.outputs, out):
                h = step.outputs[b.name]
                expected = before[b.name].reshape(h.shape).copy()
                want = np.asarray(want).reshape(h.shape)
                rows = None if h.bound is None else evaluate(h.rows_bound(), vals)
                if type(op).__name__ == "Copy":
                    r0, n = bound.get("dst_row", 0), bound.get("valid", op.rows)
                    expected[r0 : r0 + n] = want[r0 : r0 + n]
                elif rows is None or not h.shape:
                    expected[...] = want
                else:
                    expected[:rows] = want[:rows]
                got = torch_to_numpy(self._view(h)).reshape(h.shape)
                sel = slice(None) if rows is None or not h.shape or type(op).__name__ == "Copy" else slice(0, rows)
                verdict = compare(got[sel], expected[sel], tol,
                                  bound=None if bound_fn is None else np.asarray(bound_fn).reshape(h.shape)[sel])
                if not verdict:
                    raise StepCheckFailed(f"step {step.name}, output {b.name}: {verdict.detail}")

    def __call__(self, *arrays, **values):
        torch = self._torch
        from ..tensor import capturing, numpy_to_torch

        rec = self.recording
        inputs, value_params = self.graph._parameters()
        vals = _check_values(self.graph.name, value_params, values)
        given = [a for a in arrays if a is not None]
        if len(given) != len(rec.inputs):
            raise TypeError(f"{self.graph.name} takes {len(rec.inputs)} inputs, got {len(given)}")
        for (name, h), a in zip(rec.inputs.items(), given):
            a = np.asarray(a)
            if tuple(a.shape) != tuple(h.shape):
                raise ValueError(f"{name} is {tuple(a.shape)}, this version was compiled for {tuple(h.shape)}: "
                                 f"a new shape is a new compile")
            if np.dtype(a.dtype) != np.dtype(h.dtype):
                raise TypeError(f"{name} is {a.dtype}, this version takes {np.dtype(h.dtype)}")
        rec.check_limits(vals)   # out-of-range indices are refused before any dispatch
        for (name, h), a in zip(rec.inputs.items(), given):
            self.tensors[h.buffer.name].copy_(numpy_to_torch(np.asarray(a).reshape(-1), self.device))
        i = self._ring_at
        self._ring_at = (i + 1) % len(self._ring)
        if self._ring_done[i] is not None:
            self._ring_done[i].synchronize()
        for e, slot in self._slots.items():
            self._ring[i][slot] = evaluate(e, vals)
        self._values.copy_(self._ring[i], non_blocking=True)
        done = torch.cuda.Event()
        done.record()
        self._ring_done[i] = done
        if self.check:
            self._launch_checked(vals)
        elif self._cuda_graph is None:
            self._launch_all()                      # warm-up outside capture
            torch.cuda.synchronize()
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            g = torch.cuda.CUDAGraph()
            with capturing(g, stream=side):
                self._launch_all()
            torch.cuda.current_stream().wait_stream(side)
            self._cuda_graph = g   # capture records, it does not run: this call's results are the warm-up's
        else:
            self._cuda_graph.replay()
        outs = rec.outputs
        result = tuple(DeviceBuffer(self._view(h)) for h in outs) if isinstance(outs, tuple) else (
            None if outs is None else DeviceBuffer(self._view(outs)))
        if rec.carried is None:
            return result
        carried = {}
        for name, v in rec.carried.values.items():
            carried[name] = int(self._view(v).reshape(-1)[0].item()) if isinstance(v, Handle) else evaluate(v, vals)
        return carried if result is None else (*result, carried) if isinstance(result, tuple) else (result, carried)

    def read(self, held: Held) -> np.ndarray:
        """A state's (or weight's) current contents."""
        from ..tensor import torch_to_numpy

        for b in self.recording.buffers:
            if b.held is held:
                return torch_to_numpy(self.tensors[b.name]).reshape(b.shape)
        raise KeyError("this version does not hold that buffer")

    def write(self, held: Held, array: np.ndarray) -> None:
        from ..tensor import numpy_to_torch

        for b in self.recording.buffers:
            if b.held is held:
                self.tensors[b.name].copy_(numpy_to_torch(np.asarray(array).reshape(-1).astype(b.dtype), self.device))
                return
        raise KeyError("this version does not hold that buffer")

    def release(self) -> None:
        self._cuda_graph = None
        self.tensors = {}
