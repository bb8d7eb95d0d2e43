"""Re-export of ``iron_b200.declare`` under the reference's module path."""

from iron_b200.declare import *  # noqa: F401,F403


def __getattr__(name):
    import iron_b200.declare as d

    return getattr(d, name)
