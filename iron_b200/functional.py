"""Functions for a graph's body, under ``torch.nn.functional``'s names.

Each records the operator steps that compute it and returns their handle
(iron/functional.py:30-180).  Weights are a checkpoint's ``(out, in)``, as
``torch.nn.Linear`` stores them.
"""

from __future__ import annotations

import dataclasses
import math

import ml_dtypes

from .graph.handle import Handle, State
from .lm.config import Precision
from .operators.causal_conv import CausalConv1d
from .operators.copy import Copy
from .operators.flm.gemm.design import Epilogue
from .operators.flm.gemm.op import ProjectionGEMM
from .operators.gemm import GEMM
from .operators.gelu import GELU
from .operators.gemv import GEMV
from .operators.layer_norm import LayerNorm
from .operators.rms_norm import RMSNorm
from .operators.rope import RoPE
from .operators.silu import SiLU


def linear(x, weight, bias=None, *, precision: Precision = Precision.MEDIUM, **gemv) -> Handle:
    """``x @ weight.T`` plus ``bias`` on every row if given.

    One row runs on GEMV; several rows run on ProjectionGEMM at ``precision``, or on GEMM at
    ``Precision.HIGHEST`` (iron/functional.py:30-64).
    """
    if len(x.shape) not in (1, 2):
        raise ValueError(f"linear(): x {tuple(x.shape)} is not (in,) or (rows, in)")
    one_row = len(x.shape) == 1 or x.shape[0] == 1
    if one_row:
        y = GEMV.step(weight, x.reshape(x.shape[-1]), **gemv)
        if len(x.shape) == 2:
            y = y.reshape(1, y.shape[0])
    elif gemv:
        raise ValueError(f"linear(): {x.shape[0]} rows take no GEMV {sorted(gemv)}")
    elif precision == Precision.HIGHEST:
        y = GEMM.step(x, weight, b_col_maj=True, precision=Precision.HIGHEST)
    else:
        y = ProjectionGEMM.step(x, weight, b_col_maj=True, epilogue_modes=(Epilogue.NONE,), precision=precision)
    if bias is None:
        return y
    rows = math.prod(y.shape) // bias.shape[0]
    return (y.reshape(rows, bias.shape[0]) + bias).reshape(y.shape)


def _last_axis(name: str, x, normalized_shape) -> None:
    given = (normalized_shape,) if isinstance(normalized_shape, int) else tuple(normalized_shape)
    if given != tuple(x.shape[-1:]):
        raise ValueError(f"{name}(): normalized_shape {list(given)} is not the last axis of input "
                         f"{list(x.shape)}; only ({x.shape[-1]},) is normalized")


def rms_norm(x, normalized_shape, weight=None, eps: float | None = None) -> Handle:
    """``x`` over the RMS of its last axis, times ``weight`` if given (``eps`` None: the dtype's epsilon)."""
    _last_axis("rms_norm", x, normalized_shape)
    if eps is None:
        eps = float(ml_dtypes.finfo(x.dtype).eps)
    shape = x.shape
    rows = math.prod(shape) // shape[-1]
    y = RMSNorm.step(x.reshape(rows, shape[-1]), weight=weight, epsilon=eps)
    return y.reshape(shape)


def layer_norm(x, normalized_shape, weight=None, bias=None, eps: float = 1e-5) -> Handle:
    """``x`` minus its mean over its standard deviation along the last axis (``eps`` under the
    root), times ``weight`` and plus ``bias`` when given (iron/functional.py:97-110)."""
    _last_axis("layer_norm", x, normalized_shape)
    shape = x.shape
    rows = math.prod(shape) // shape[-1]
    y = LayerNorm.step(x.reshape(rows, shape[-1]), weight=weight, epsilon=eps)
    if bias is not None:
        y = y + bias
    return y.reshape(shape)


def gelu(x, approximate: str = "none") -> Handle:
    """GELU, exact by default; ``approximate="tanh"`` for the tanh form (iron/functional.py:118-124)."""
    shape = x.shape
    return GELU.step(x.reshape(math.prod(shape)), approximate=approximate).reshape(shape)


def silu(x) -> Handle:
    """``x * sigmoid(x)``."""
    shape = x.shape
    return SiLU.step(x.reshape(math.prod(shape))).reshape(shape)


def rope(x, angles) -> Handle:
    """``x`` ``(rows, head_dim)`` turned by RoPE, each angle row serving ``rows / angle_rows`` rows."""
    return RoPE.step(x, angles)


@dataclasses.dataclass(frozen=True)
class ConvState:
    """What a short causal conv carries between calls (iron/functional.py:130-144)."""

    read: Handle
    write: Handle
    window: State | None = None
    tail: State | None = None


def causal_conv1d(x, taps, state: ConvState) -> Handle:
    """``x`` ``(rows, channels)`` through a depth-wise causal filter of ``K`` taps.

    Output row ``t`` is ``sum_k taps[k] * x[t - K + 1 + k]``; the ``K - 1`` rows before
    ``x``'s first come from ``state.read`` and the ``K - 1`` rows ending this call go to
    ``state.write`` (iron/functional.py:147-180).  ``x`` bounded per call (``x[:n]``) is a
    prompt chunk; otherwise it is one row, a decode step.  The reference stages the rows in
    ``state.window`` and ``state.tail``; one fused step needs neither, so both may be None.
    """
    decode = x.bound is None
    if decode and x.shape[0] != 1:
        raise ValueError(f"causal_conv1d(): x {tuple(x.shape)} is neither bounded per call nor one row")
    y, _ = CausalConv1d.step(x, taps, state.read, new_history=state.write, decode=decode)
    return y
