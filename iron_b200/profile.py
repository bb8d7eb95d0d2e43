"""Profiles: tunable values keyed by operator shape, applied as an operator is made.

The contract of ``iron/common/declare/profile.py:25-177``: a profile is a list of entries
``(operator class, dimensions to match, tunables to give)``.  When an operator is constructed
through a profile, each tunable the caller left open takes the value of the most specific
entry that matches the call's dimensions -- an entry that names more dimensions is more
specific, an entry for a base class serves its subclasses, and two equally specific entries
that disagree are an error, not a silent pick.  What the caller gives always wins and is
remembered as ``pinned``.  Profiles are JSON, ``{"entries": [{"operator": name, ...}, ...]}``,
one entry per line when written.

On B200 the tunables are not AIE tile sizes but the launch choices of the CUDA kernels (the
key split of the decode attention, ...); the AIE tunables of a reference profile are still
accepted, since the operator classes declare them, and ignored by the launches.
"""

from __future__ import annotations

import json
import types
from dataclasses import MISSING
from enum import Enum
from pathlib import Path
from typing import Any, Iterator, Mapping


class Profile:
    """Entries ``(cls, dims, tunables)``; see the module docstring."""

    def __init__(self) -> None:
        self._entries: list[tuple[type, dict[str, Any], dict[str, Any]]] = []

    # ---- building ----
    def add(self, cls: type, **fields: Any) -> None:
        """One entry for ``cls``: its params are dimensions to match (a param left out matches
        any value), its tunables the values to give.  ``TypeError`` for a name the class does
        not declare, for a tunable the class fixes itself, or for an entry giving no tunable."""
        decl = cls.declaration
        dims: dict[str, Any] = {}
        gives: dict[str, Any] = {}
        for name, value in fields.items():
            if name in decl.tunables:
                if not decl.tunables[name].init:
                    raise TypeError(f"{cls.__name__}.{name} is fixed by the class, not a tunable a profile gives")
                gives[name] = value
            elif name in decl.params:
                if decl.params[name].derive is not None:
                    raise TypeError(f"{cls.__name__}.{name} is derived, not a dimension a profile matches")
                dims[name] = value
            else:
                raise TypeError(f"{cls.__name__} declares no field {name!r}")
        if not gives:
            raise TypeError(f"an entry for {cls.__name__} must give a tunable")
        self._entries.append((cls, dims, gives))

    # ---- applying ----
    @staticmethod
    def dims(cls: type, given: Mapping[str, Any]) -> dict[str, Any]:
        """Every dimension a ``cls(**given)`` call constructs with: what it gives, else a plain
        default; one that is derived or defaults from other fields is unknown (None) until the
        operator exists, so an entry naming it matches only a call that gives it."""
        out: dict[str, Any] = {}
        for name, f in cls.declaration.params.items():
            if f.kind == "tunable":
                continue
            if name in given:
                out[name] = given[name]
            elif f.derive is not None or isinstance(f.default, types.FunctionType):
                out[name] = None
            elif f.default is not MISSING:
                out[name] = f.default
        return out

    @staticmethod
    def matches(entry_dims: Mapping[str, Any], dims: Mapping[str, Any]) -> bool:
        return all(name in dims and dims[name] == value for name, value in entry_dims.items())

    def tunables_for(self, cls: type, given: Mapping[str, Any]) -> dict[str, Any]:
        """The tunables this profile gives a ``cls(**given)`` call, each from the most specific
        matching entry; ``ValueError`` when two entries of equal specificity disagree."""
        dims = self.dims(cls, given)
        best: dict[str, tuple[int, Any]] = {}
        for base, entry_dims, gives in self._entries:
            if not issubclass(cls, base) or not self.matches(entry_dims, dims):
                continue
            rank = len(entry_dims)
            for name, value in gives.items():
                held = best.get(name)
                if held is None or rank > held[0]:
                    best[name] = (rank, value)
                elif rank == held[0] and held[1] != value:
                    raise ValueError(f"profile is ambiguous for {cls.__name__} {dims}: {name}={held[1]} and "
                                     f"{name}={value} from entries of equal specificity")
        return {name: value for name, (_, value) in best.items()}

    def make(self, cls: type, **kwargs: Any):
        """``cls(**kwargs)`` with its open tunables filled from this profile; the tunables the
        caller gave stay the caller's (``op.pinned``)."""
        given = {name: value for name, value in kwargs.items() if value is not None}
        pinned = {name for name in given if name in cls.declaration.tunables}
        op = cls(**{**self.tunables_for(cls, given), **given})
        op.pinned = pinned
        return op

    # ---- files ----
    @classmethod
    def load(cls, path) -> "Profile":
        """The profile ``save`` wrote.  ``ValueError`` for a file of another form or an operator
        the catalogue does not hold."""
        from .operators import CATALOG

        CATALOG = {op.__name__: op for op in CATALOG}
        data = json.loads(Path(path).read_text())
        if not isinstance(data, dict) or set(data) != {"entries"}:
            raise ValueError(f"{path}: a profile is {{'entries': [...]}}")
        profile = cls()
        for entry in data["entries"]:
            fields = dict(entry)
            name = fields.pop("operator", None)
            if name not in CATALOG:
                raise ValueError(f"{path}: no operator {name!r} in the catalogue")
            op_cls = CATALOG[name]
            for key, f in op_cls.declaration.params.items():   # an Enum-valued field is its member's value in JSON
                if key in fields and isinstance(f.domain, type) and issubclass(f.domain, Enum):
                    fields[key] = f.domain(fields[key])
            profile.add(op_cls, **fields)
        return profile

    def save(self, path) -> None:
        from .operators import CATALOG

        names = {op: op.__name__ for op in CATALOG}
        lines = []
        for op, dims, gives in self._entries:
            if op not in names:
                raise ValueError(f"{op.__qualname__} is not in the catalogue")
            plain = {k: (v.value if isinstance(v, Enum) else v) for k, v in {**dims, **gives}.items()}
            lines.append(json.dumps({"operator": names[op], **plain}))
        Path(path).write_text('{"entries": [\n  ' + ",\n  ".join(lines) + "\n]}\n")

    def __iter__(self) -> Iterator[tuple[type, dict[str, Any], dict[str, Any]]]:
        return iter(self._entries)

    def __len__(self) -> int:
        return len(self._entries)

    def __repr__(self) -> str:
        return f"Profile({', '.join(dict.fromkeys(op.__name__ for op, _, _ in self._entries))})"
