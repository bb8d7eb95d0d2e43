"""The per-operator parity harness: cases, seeded vectors, dispatch, judgement, timing.

Mirrors ``iron/common/testing.py`` (``Case`` :34-54, ``Testing`` :60-81, ``vectors`` :95-144,
``run_test`` :224-297, ``time_call`` :172-221): every operator class carries
``test = Testing(cases, draw=...)``; ``run_test`` constructs the operator, draws inputs with
``default_rng(seed)``, runs it on the device and judges each output against
``op.reference()`` under ``op.tolerance()``.
"""

from __future__ import annotations

import dataclasses
import statistics
from typing import Any, Callable, Iterable, Mapping

import numpy as np
from ml_dtypes import bfloat16

from .declare import Buffer, Operator
from .verify import Verdict


@dataclasses.dataclass(frozen=True)
class Case:
    """One construction of an operator."""

    kwargs: dict = dataclasses.field(default_factory=dict)
    extensive: bool = False
    id: str | None = None
    bench: bool = False
    lower: bool = False

    @property
    def label(self) -> str:
        return self.id or "-".join(f"{k}_{v}" for k, v in self.kwargs.items())


@dataclasses.dataclass(frozen=True)
class Testing:
    """How an operator is checked: its cases and how its inputs are drawn."""

    __test__ = False

    cases: Any
    draw: Callable[[Any], dict] | None = None

    def resolve(self, cls: type, dev=None) -> list[Case]:
        out = []
        for c in [self.cases] if callable(self.cases) else self.cases:
            out += list(c(cls, dev)) if callable(c) else [c]
        return out


@dataclasses.dataclass
class Vectors:
    inputs: dict[str, np.ndarray]
    outputs: dict[str, np.ndarray]

    def __getitem__(self, name: str) -> np.ndarray:
        return self.inputs[name] if name in self.inputs else self.outputs[name]


def vectors(op: Operator, *, seed: int = 42, scale: float = 4.0, normal: Iterable[Buffer] = (),
            centered: Iterable[Buffer] = (), given: Mapping[Buffer, Any] | None = None) -> Vectors:
    """Random inputs for ``op``'s declared buffers and the reference's outputs for them.

    Uniform on ``[0, scale)`` by default, ``normal`` inputs ``N(0, scale)``, ``centered`` ones
    shifted by ``-scale/2``, integer buffers uniform integers on ``[0, scale]``; ``given``
    supplies an array (or a shape to draw) per input.
    """
    given_names = {o.name: v for o, v in (given or {}).items()}
    normal_names = {o.name for o in normal}
    centered_names = {o.name for o in centered}
    unknown = (given_names.keys() | normal_names | centered_names) - {b.name for b in op.inputs}
    if unknown:
        raise ValueError(f"{type(op).__name__} has no input {sorted(unknown)}")
    rng = np.random.default_rng(seed)
    inputs = {}
    for b in op.inputs:
        value = given_names.get(b.name)
        if isinstance(value, np.ndarray):
            inputs[b.name] = value
            continue
        shape = b.host_shape if value is None else tuple(value)
        dtype = np.dtype(bfloat16 if b.dtype is None else b.host_dtype)
        if dtype.kind not in "fc" and dtype != bfloat16:
            t = rng.integers(0, int(scale) + 1, shape).astype(dtype)
        else:
            draw = rng.standard_normal if b.name in normal_names else rng.random
            t = (draw(shape) * scale).astype(dtype)
            if b.name in centered_names:
                t = (t.astype(np.float32) - scale / 2).astype(dtype)
        inputs[b.name] = t
    return Vectors(inputs, op._call_reference(inputs))


def time_call(fn: Callable[[], None], repeats: int = 20, warmup: int = 3) -> dict[str, float]:
    """Median and MAD (microseconds) of ``repeats`` device-timed calls after ``warmup``."""
    import torch

    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(repeats):
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        fn()
        stop.record()
        stop.synchronize()
        times.append(start.elapsed_time(stop) * 1e3)
    med = statistics.median(times)
    return {"median_us": med, "mad_us": statistics.median(abs(t - med) for t in times),
            "min_us": min(times), "max_us": max(times)}


def run_test(cls: type, case: Case, *, seed: int = 42, time: bool = False) -> dict[str, Any]:
    """Construct, draw, dispatch and judge one case.  Returns ``{"verdicts": ..., "timing": ...}``
    and raises ``AssertionError`` on a verdict that fails."""
    from .tensor import Tensor

    op = cls(**case.kwargs).resolved(None)
    testing: Testing = cls.test
    extra = testing.draw(op) if testing.draw else {}
    vec = vectors(op, seed=seed, **extra)
    ins = [Tensor(vec.inputs[b.name]) for b in op.inputs]
    outs = [Tensor(b.shape, dtype=b.host_dtype) for b in op.outputs if b.decl.direction == "out"]
    op(*ins, *outs)
    written = {b.name: t.numpy() for b, t in zip([b for b in op.outputs if b.decl.direction == "out"], outs)}
    for b, t in zip(op.inputs, ins):
        if b.decl.direction == "inout":
            written[b.name] = t.numpy()
    tol = op.tolerance()
    verdicts: dict[str, Verdict] = {}
    if tol is not None:
        verdicts = op.judge(vec.inputs, written, tol, expected=vec.outputs)
        bad = {n: v.detail for n, v in verdicts.items() if not v}
        assert not bad, f"{cls.__name__}({case.label}): {bad}"
    result: dict[str, Any] = {"verdicts": verdicts, "op": op}
    if time:
        t = time_call(lambda: op(*ins, *outs))
        result["timing"] = t
        try:
            result["throughput_gops"] = op.ops() / (t["median_us"] * 1e3)
        except NotImplementedError:
            pass
    return result
