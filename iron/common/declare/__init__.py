"""``iron.common.declare``: the declaration vocabulary (iron/common/declare/__init__.py), one
module in ``iron_b200`` and a package in the reference; its sub-modules re-export from there."""

from iron_b200.declare import *  # noqa: F401,F403
from iron_b200.declare import Operator, graph_recorder  # noqa: F401
from iron_b200.lm.config import Precision  # noqa: F401


def __getattr__(name):
    import iron_b200.declare as d

    return getattr(d, name)
