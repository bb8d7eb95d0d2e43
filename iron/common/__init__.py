"""``iron.common``: the names the reference's model code takes from it (iron/common/__init__.py):
``Precision`` and ``Profile``; its sub-packages ``graph``, ``declare``, ``testing`` resolve through
the alias finder of ``iron``."""

import importlib


def __getattr__(name):
    if name == "Precision":
        return importlib.import_module("iron_b200.lm.config").Precision
    if name == "Profile":
        return importlib.import_module("iron_b200.declare").Profile
    if name in ("graph", "declare", "testing", "elementwise"):
        return importlib.import_module(f"iron.common.{name}")
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
