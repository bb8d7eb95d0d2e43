"""``iron``: the reference's import paths over the B200 package.

Code written against amd/IRON imports ``iron``, ``iron.functional``, ``iron.lm``,
``iron.operators.<name>``, ``iron.common.graph``, ``iron.common.declare`` ... (iron/__init__.py:29-47,
iron/lm/__init__.py:46-94, iron/functional.py:16-27).  This package makes those paths resolve to
``iron_b200``'s modules, the very same module objects, so a model file of the reference --
``iron/applications/llama/model.py``, ``granite/model.py``, ``granite_hybrid/model.py`` -- imports
and runs unchanged on the B200 kernels.  Nothing is reimplemented here: a finder on
``sys.meta_path`` maps a module name to its ``iron_b200`` counterpart on first import.

    iron.<x>                         ->  iron_b200.<x>            (functional, lm, operators, applications, ...)
    iron.common.graph[.<x>]          ->  iron_b200.graph[.<x>]
    iron.common.declare[.<x>]        ->  re-exports of iron_b200.declare (one module here, a package there)
    iron.common.testing              ->  iron_b200.testing
    iron.common.elementwise          ->  iron_b200.elementwise
    iron.common                      ->  this package's ``common`` namespace (Precision, Profile)

The names ``iron`` itself exports are loaded on first use, so ``import iron`` stays light (no
torch, no CUDA), as iron/tests/infrastructure/test_no_torch_on_import.py asks of the reference.
"""

from __future__ import annotations

import importlib
import importlib.abc
import importlib.util
import sys

__all__ = ["Carried", "CarriedLoop", "CompiledGraph", "Graph", "Precision", "Profile", "Scratchpad",
           "carry", "clamp", "on_host", "param", "state", "weight"]

#: reference module path (prefix) -> module here; the longest prefix wins, the rest of the path is kept
_PREFIXES = {
    "iron.common.graph": "iron_b200.graph",
    "iron.common.testing": "iron_b200.testing",
    "iron.common.elementwise": "iron_b200.elementwise",
    "iron.common.image.allocator": "iron_b200.arena",
    "iron": "iron_b200",
}
#: modules that are one file here where the reference has a package: sub-paths collapse onto them
_FLAT = ("iron_b200.testing", "iron_b200.elementwise", "iron_b200.arena")


def _target(name: str) -> str | None:
    if name == "iron.common":
        return None   # a namespace of this package (below)
    for prefix in sorted(_PREFIXES, key=len, reverse=True):
        if name == prefix or name.startswith(prefix + "."):
            mapped = _PREFIXES[prefix] + name[len(prefix):]
            for flat in _FLAT:
                if mapped.startswith(flat + "."):
                    return flat
            return mapped
    return None


class _AliasLoader(importlib.abc.Loader):
    def __init__(self, target: str):
        self.target = target

    def create_module(self, spec):
        module = importlib.import_module(self.target)   # the module object itself, not a copy
        self.own_spec = module.__spec__
        return module

    def exec_module(self, module):
        # the import system has just stamped the alias's spec on the module: put its own back, so
        # that its relative imports keep resolving against the package it lives in
        module.__spec__ = self.own_spec


class _AliasFinder(importlib.abc.MetaPathFinder):
    def find_spec(self, name, path=None, target=None):
        if not name.startswith("iron.") or name == "iron.common" or name.startswith("iron.common.declare"):
            return None
        mapped = _target(name)
        if mapped is None:
            return None
        try:
            found = importlib.util.find_spec(mapped)
        except (ImportError, ValueError):
            found = None
        if found is None:
            return None
        spec = importlib.util.spec_from_loader(name, _AliasLoader(mapped), is_package=found.submodule_search_locations is not None)
        return spec


if not any(isinstance(f, _AliasFinder) for f in sys.meta_path):
    sys.meta_path.insert(0, _AliasFinder())

_LAZY = {
    "Precision": ("iron_b200.lm.config", "Precision"),
    "Profile": ("iron_b200.declare", "Profile"),
    "on_host": ("iron_b200.graph", "on_host"),
    "CarriedLoop": ("iron_b200.graph", "CarriedLoop"),
}


def __getattr__(name):
    if name in _LAZY:
        module, attr = _LAZY[name]
        return getattr(importlib.import_module(module), attr)
    if name in __all__:
        return getattr(importlib.import_module("iron_b200.graph"), name)
    if name in ("functional", "lm", "operators", "applications", "common"):
        return importlib.import_module(f"iron.{name}")
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")


def __dir__():
    return sorted(set(globals()) | set(__all__))
