"""Static planning of one device arena shared by every compiled version of a graph.

What the reference does with ``Pool.place`` / ``ArenaPlan.place_image``
(iron/common/image/allocator.py:143-227) for the NPU's scratch arena, planned here for
one HBM allocation per model:

* a *resident* (weight, state such as a KV cache) gets one offset the first time any
  version names it and keeps it in every later version, so a prompt-chunk graph and a
  decode-step graph see the same caches;
* a *transient* (an intermediate) only needs its bytes between its first and last use;
  transients are placed largest first into the tightest gap that is free of the
  residents and of every transient whose live range overlaps theirs;
* nothing placed ever moves.

Offsets are multiples of 256 bytes (every kernel here wants 16- or 32-byte aligned rows;
256 keeps TMA descriptors and 256-bit loads legal for any row slice).  The NPU's
3.5 GiB bank rule has no counterpart in HBM and is not reproduced.
"""

from __future__ import annotations

import dataclasses
from typing import Hashable, Iterable, Mapping

ALIGN = 256


def align_up(x: int, a: int = ALIGN) -> int:
    return -(-x // a) * a


@dataclasses.dataclass(frozen=True)
class Span:
    """A placed buffer: ``size`` bytes at ``offset`` of the arena."""

    name: str
    offset: int
    size: int

    @property
    def end(self) -> int:
        return self.offset + self.size

    def overlaps(self, other: "Span") -> bool:
        return self.offset < other.end and other.offset < self.end


@dataclasses.dataclass(frozen=True)
class Live:
    """The steps (inclusive) between which a transient's bytes must survive."""

    first: int
    last: int

    def overlaps(self, other: "Live") -> bool:
        return self.first <= other.last and other.first <= self.last


def live_ranges(steps: Iterable[Iterable[str]], names: Iterable[str]) -> dict[str, Live]:
    """The live range of each of ``names`` over ``steps`` (each step: the buffers it touches).

    A buffer no step touches is live for the whole run (it is an input or an output the
    caller reads afterwards).
    """
    names = list(names)
    seen: dict[str, list[int]] = {}
    count = 0
    for i, touched in enumerate(steps):
        count = i + 1
        for n in touched:
            seen.setdefault(n, []).append(i)
    out = {}
    for n in names:
        at = seen.get(n)
        out[n] = Live(at[0], at[-1]) if at else Live(0, max(count - 1, 0))
    return out


def place(ranges: Mapping[str, Live], sizes: Mapping[str, int], fixed: Iterable[Span] = (),
          align: int = ALIGN) -> tuple[dict[str, Span], int]:
    """Place transients; return their spans and the top byte used."""
    fixed = list(fixed)
    placed: list[tuple[Span, Live]] = []
    order = sorted(ranges, key=lambda n: (-sizes[n], ranges[n].first, n))
    for name in order:
        live, size = ranges[name], sizes[name]
        walls = sorted([*fixed, *(s for s, r in placed if r.overlaps(live))], key=lambda s: s.offset)
        cursor, best, best_gap = 0, None, None
        for wall in walls:
            at = align_up(cursor, align)
            gap = wall.offset - at
            if gap >= size and (best_gap is None or gap < best_gap):
                best, best_gap = at, gap
            cursor = max(cursor, align_up(wall.end, align))
        offset = align_up(cursor, align) if best is None else best
        placed.append((Span(name, offset, size), live))
    spans = {s.name: s for s, _ in placed}
    return spans, max((s.end for s in spans.values()), default=0)


class ArenaPlan:
    """Offsets for every buffer of every version compiled against one arena."""

    def __init__(self, align: int = ALIGN):
        self.align = align
        self._residents: dict[Hashable, Span] = {}
        self._size = 0

    @property
    def size(self) -> int:
        return self._size

    @property
    def residents(self) -> dict[Hashable, Span]:
        return dict(self._residents)

    def resident(self, key: Hashable, size: int, name: str | None = None) -> Span:
        """The span of resident ``key``, placed above everything on first sight."""
        held = self._residents.get(key)
        if held is None:
            held = Span(name or str(key), align_up(self._size, self.align), size)
            self._residents[key] = held
            self._size = held.end
        elif held.size != size:
            raise ValueError(
                f"resident {name or key!r} is {size} bytes here but was placed with "
                f"{held.size}; one storage is one size in every version")
        return held

    def place_version(self, steps: Iterable[Iterable[str]], sizes: Mapping[str, int],
                      residents: Mapping[str, Hashable]) -> dict[str, Span]:
        """Place one version's buffers: ``residents`` by storage key, the rest by live range."""
        unknown = set(residents) - set(sizes)
        if unknown:
            raise ValueError(f"residents {sorted(unknown)} have no size")
        out = {}
        for name, key in residents.items():
            held = self.resident(key, sizes[name], name)
            out[name] = Span(name, held.offset, held.size)
        steps = [list(s) for s in steps]
        ranges = live_ranges(steps, (n for n in sizes if n not in residents))
        spans, top = place(ranges, sizes, fixed=self._residents.values(), align=self.align)
        self._size = max(self._size, top)
        out.update(spans)
        return out
