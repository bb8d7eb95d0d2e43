"""iron_b200: the operator hot path of amd/IRON as hand-written sm_100a CUDA kernels.

The public names mirror ``iron/__init__.py:29-47``: ``Graph``, ``param``, ``state``,
``weight``, ``carry``, ``clamp``, ``Scratchpad``, ``Carried``, ``Precision`` and
``iron_b200.functional``.  Nothing here imports torch until a device is needed, so the
declaration layer, the recorder and the host references import on a machine without one.
"""

from .graph import (Carried, CompiledGraph, Graph, Handle, Scratchpad, carry, clamp, param, state, weight)
from .lm.config import Precision

__all__ = ["Graph", "CompiledGraph", "Handle", "param", "state", "weight", "carry", "clamp", "Scratchpad",
           "Carried", "Precision"]
