"""Graphs: bodies recorded on handles, compiled to CUDA graphs over one device arena."""

from .compiled import Carried, CompiledGraph, Graph, Scratchpad, StepCheckFailed, walk
from .expr import Expr, clamp
from .handle import Handle, Param, State, Weight, param, state, weight
from .record import Carry, Recorder, Recording, Step, carry

__all__ = ["Graph", "CompiledGraph", "Scratchpad", "Carried", "StepCheckFailed", "walk", "Expr", "clamp", "Handle", "Param",
           "State", "Weight", "param", "state", "weight", "Carry", "carry", "Recorder", "Recording", "Step"]
