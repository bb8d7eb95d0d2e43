"""Tolerances and the comparison an operator's output is judged by.

The reference takes ``Tolerance``/``compare``/``Verdict`` from mlir-aie
(``aie.utils.verify``); their semantics are pinned by the reference's own tests
(iron/tests/common/test_judging.py:138-174, iron/tests/support/judging.py:24-84) and
restated here:

* ``relative(rtol, atol, range_frac)`` admits ``|a-b| < rtol*(|a|+|b|)``, or
  ``|a-b| < atol`` (float32's tiny when None), or ``|a-b| <= range_frac*max|ref|``;
* ``bounded(fn)`` admits ``|a-b| <= fn(*inputs)`` elementwise;
* ``bf16_ulps(n, atol)`` admits ``n`` bf16 steps either side of the rounded reference;
* ``exact()`` admits only the reference cast to the output's dtype;
* ``max_mismatch_frac`` lets that share of the elements fail;
* a NaN where the reference is finite always fails.
"""

from __future__ import annotations

import dataclasses
from typing import Callable

import numpy as np
from ml_dtypes import bfloat16


def round_to(x, dtype):
    """``x`` rounded to ``dtype`` (nearest even), as float64."""
    return np.asarray(x, np.float64).astype(np.float32).astype(dtype).astype(np.float64)


@dataclasses.dataclass(frozen=True)
class Tolerance:
    """How far an output may lie from its reference.  ``kind`` picks the test."""

    rtol: float | None = None
    atol: float | None = None
    max_mismatch_frac: float = 0.0
    note: str = ""
    kind: str = "relative"
    ulps: int | None = None
    range_frac: float | None = None
    bound: Callable | None = None

    @classmethod
    def exact(cls, note: str = "") -> "Tolerance":
        return cls(kind="exact", note=note)

    @classmethod
    def relative(cls, rtol, atol=None, range_frac=None, note: str = "") -> "Tolerance":
        return cls(rtol=rtol, atol=atol, range_frac=range_frac, note=note, kind="relative")

    @classmethod
    def bf16_ulps(cls, n: int, atol=None, note: str = "") -> "Tolerance":
        return cls(ulps=n, atol=atol, note=note, kind="ulps")

    @classmethod
    def bounded(cls, bound_fn, note: str = "", max_mismatch_frac: float = 0.0) -> "Tolerance":
        return cls(bound=bound_fn, note=note, kind="bound", max_mismatch_frac=max_mismatch_frac)


@dataclasses.dataclass(frozen=True)
class Verdict:
    """The outcome of one comparison; truthy when it passed."""

    ok: bool
    n_mismatch: int
    n_checked: int
    detail: str = ""

    def __bool__(self) -> bool:
        return self.ok


def _bf16_steps(x: np.ndarray, n: int, toward) -> np.ndarray:
    out = x.astype(bfloat16)
    for _ in range(n):
        out = np.nextafter(out, np.asarray(toward, bfloat16))
    return out.astype(np.float64)


def compare(actual, expected, tolerance: Tolerance, bound=None) -> Verdict:
    """Judge ``actual`` against ``expected`` under ``tolerance``.

    ``bound`` is the evaluated error bound of a ``bounded`` tolerance (an array
    broadcastable to the output).
    """
    a = np.asarray(actual).astype(np.float64).reshape(-1)
    tol = tolerance
    out_dtype = np.asarray(actual).dtype
    if tol.kind == "ulps":
        e = round_to(np.asarray(expected).reshape(-1), bfloat16)
    elif tol.kind == "exact":
        e = np.asarray(expected).astype(out_dtype).astype(np.float64).reshape(-1)
    else:
        e = np.asarray(expected).astype(np.float32).astype(np.float64).reshape(-1)
    if a.shape != e.shape:
        return Verdict(False, max(a.size, e.size), max(a.size, e.size),
                       f"shape {np.shape(actual)} against {np.shape(expected)}")
    diff = np.abs(a - e)
    both_nan = np.isnan(a) & np.isnan(e)
    same_inf = np.isinf(a) & np.isinf(e) & (a == e)
    if tol.kind == "exact":
        ok = a == e
    elif tol.kind == "bound":
        if bound is None:
            raise TypeError("a bounded tolerance needs its evaluated bound")
        b = np.broadcast_to(np.ravel(np.asarray(bound, np.float64)), a.shape)
        ok = diff <= b
    elif tol.kind == "ulps":
        ok = (a >= _bf16_steps(e, tol.ulps or 0, -np.inf)) & (a <= _bf16_steps(e, tol.ulps or 0, np.inf))
        if tol.atol is not None:
            ok |= diff < tol.atol
    else:
        floor = float(np.finfo(np.float32).tiny) if tol.atol is None else tol.atol
        ok = (diff < (tol.rtol or 0.0) * (np.abs(a) + np.abs(e))) | (diff < floor) | (diff == 0)
    if tol.range_frac is not None and tol.kind in ("relative", "ulps"):
        finite = np.isfinite(e)
        scale = float(np.max(np.abs(e[finite]))) if finite.any() else 0.0
        ok |= diff <= tol.range_frac * scale
    ok = np.where(np.isnan(diff), False, ok) | both_nan | same_inf
    n_bad = int((~ok).sum())
    allowed = int(tol.max_mismatch_frac * a.size)
    detail = ""
    if n_bad:
        worst = int(np.nanargmax(np.where(ok, -1.0, np.where(np.isnan(diff), np.inf, diff))))
        detail = (f"{n_bad}/{a.size} outside tolerance; worst at {worst}: "
                  f"got {a[worst]!r}, want {e[worst]!r}")
    return Verdict(n_bad <= allowed, n_bad, int(a.size), detail)
