"""A model's weights from disk to HBM.

``Checkpoint`` maps a ``.safetensors`` file (or every shard a
``model.safetensors.index.json`` names) and exposes the tensors as lazy read-only numpy
views by their own dotted names, or as a tree: ``model.layers.3.self_attn.q_proj.weight``
is ``tree.model.layers[3].self_attn.q_proj.weight`` (iron/lm/checkpoint.py:220-294,
``nest``/``leaves``/``subtree``/``renamed`` :297-424).  ``Uploader`` is the device half the
reference keeps in ``iron/common/graph/compiled.py:866-885``: each tensor goes from the
mapping through a pinned staging ring to its arena slice on a copy stream, and the
mapping's pages are dropped as soon as the bytes are staged, so loading a checkpoint
never holds a second copy of it in host memory.

PyTorch zip checkpoints (``.pth``), which the reference also parses, are refused: the
decoder models here ship as safetensors.
"""

from __future__ import annotations

import hashlib
import json
import math
import mmap
import struct
import zipfile
from collections.abc import Iterator, Mapping
from pathlib import Path
from types import SimpleNamespace
from typing import Any

import numpy as np
from ml_dtypes import bfloat16

DTYPES = {"BF16": bfloat16, "F16": np.float16, "F32": np.float32, "I64": np.int64}
_NAMES = {np.dtype(v): k for k, v in DTYPES.items()}


def save_file(tensors: Mapping[str, np.ndarray], path, metadata: Mapping[str, str] | None = None) -> Path:
    """Write ``tensors`` as one ``.safetensors`` file: an 8-byte little-endian header length,
    the JSON header (name -> dtype, shape, byte span), then the tensors' bytes in order."""
    header: dict[str, Any] = {}
    if metadata:
        header["__metadata__"] = dict(metadata)
    at = 0
    arrays = []
    for name, t in tensors.items():
        a = np.ascontiguousarray(t)
        if a.dtype not in _NAMES:
            raise ValueError(f"{name} is {a.dtype}: safetensors here holds {sorted(DTYPES)}")
        header[name] = {"dtype": _NAMES[a.dtype], "shape": list(a.shape), "data_offsets": [at, at + a.nbytes]}
        at += a.nbytes
        arrays.append(a)
    blob = json.dumps(header, separators=(",", ":")).encode()
    blob += b" " * (-len(blob) % 8)   # keep the data 8-byte aligned
    path = Path(path)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for a in arrays:
            f.write(a.view(np.uint8).reshape(-1).data if a.size else b"")
    return path


class _Mapped:
    """One ``.safetensors`` file, mapped read-only; ``tensors`` are views into the mapping."""

    def __init__(self, path: Path):
        self.path = path
        if zipfile.is_zipfile(path):
            raise ValueError(f"{path}: a PyTorch zip checkpoint; convert it to safetensors")
        with open(path, "rb") as f:
            self._map = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ)
        whole = np.frombuffer(self._map, dtype=np.uint8)
        self._base = whole.ctypes.data
        if whole.size < 8:
            raise ValueError(f"{path}: too short for a safetensors header")
        (n,) = struct.unpack("<Q", self._map[:8])
        if 8 + n > whole.size:
            raise ValueError(f"{path}: a header of {n} bytes in a file of {whole.size}")
        header = json.loads(self._map[8 : 8 + n])
        self.metadata = header.pop("__metadata__", None) or {}
        data0 = 8 + n
        self.tensors: dict[str, np.ndarray] = {}
        for name, entry in header.items():
            kind, shape, span = entry.get("dtype"), entry.get("shape"), entry.get("data_offsets", ())
            if kind not in DTYPES:
                raise ValueError(f"{path}: {name} is {kind}")
            if shape is None or len(span) != 2:
                raise ValueError(f"{path}: {name} has no data_offsets or shape")
            lo, hi = data0 + span[0], data0 + span[1]
            dtype = np.dtype(DTYPES[kind])
            if hi - lo != dtype.itemsize * math.prod(shape) or lo < data0 or hi > whole.size:
                raise ValueError(f"{path}: {name} spans bytes {lo} to {hi}, not {kind} {shape} within the file")
            self.tensors[name] = whole[lo:hi].view(dtype).reshape(shape)

    def release(self, array: np.ndarray) -> bool:
        """Drop this process's pages under ``array`` if it views this file; a later read
        faults them back in."""
        lo = array.ctypes.data - self._base
        if not (array.flags.c_contiguous and 0 <= lo < len(self._map)) or array.nbytes == 0:
            return False
        first = lo - lo % mmap.PAGESIZE
        self._map.madvise(mmap.MADV_DONTNEED, first, lo + array.nbytes - first)
        return True


def weights_file(directory) -> Path:
    """A checkpoint directory's weights: its shard index if it has one, else ``model.safetensors``."""
    index = Path(directory) / "model.safetensors.index.json"
    return index if index.exists() else index.with_name("model.safetensors")


def filled(fill: str, named: Mapping[str, tuple[tuple[int, ...], Any]], seed: int = 0) -> dict[str, np.ndarray]:
    """Arrays made from shapes alone (iron/common/graph/fill.py:13-33): ``"random"`` draws,
    from one ``default_rng(seed)`` stream in name order, matrices ``N(0, 1) / sqrt(in)`` and
    vectors ``1 + N(0, 1) / 10`` (a bias without the one); ``"unread"`` is zeros."""
    if fill == "unread":
        return {n: np.zeros(shape, dtype) for n, (shape, dtype) in named.items()}
    rng = np.random.default_rng(seed)
    out = {}
    for n, (shape, dtype) in named.items():
        x = rng.standard_normal(shape, dtype=np.float32)
        if len(shape) >= 2:
            out[n] = (x / np.sqrt(math.prod(shape[1:]))).astype(dtype)
        else:
            out[n] = np.asarray(x / 10 + (not n.endswith("bias")), dtype)
    return out


class Checkpoint:
    """A ``.safetensors`` file, or (given its ``.safetensors.index.json``) every shard of a
    sharded checkpoint merged into one mapping, ``tensors``."""

    def __init__(self, path):
        self.path = Path(path)
        index = None
        files = [self.path]
        if self.path.suffix == ".json":
            index = json.loads(self.path.read_text())["weight_map"]
            names = sorted(set(index.values()))
            for n in names:
                if Path(n).name != n:
                    raise ValueError(f"{self.path}: {n} is not a file beside the index")
            files = [self.path.parent / n for n in names]
        self._files = [_Mapped(p) for p in files]
        self.tensors: dict[str, np.ndarray] = {}
        for f in self._files:
            if index is not None:
                named = {n for n, s in index.items() if s == f.path.name}
                if named != f.tensors.keys():
                    raise ValueError(f"{f.path}: holds {sorted(f.tensors.keys() - named)} the index does not "
                                     f"name and lacks {sorted(named - f.tensors.keys())}")
            self.tensors.update(f.tensors)

    def release(self, array: np.ndarray) -> None:
        """Drop the pages of ``array`` if it views one of the files; anything else is left alone."""
        for f in self._files:
            if f.release(array):
                return

    def fingerprint(self) -> str:
        """A digest of each tensor's name, type, shape and first and last 4 KiB: what tells a
        fine-tune from its base without reading either whole."""
        h = hashlib.sha256()
        for name, t in self.tensors.items():
            n = 4096 // t.itemsize
            flat = t.reshape(-1)
            h.update(f"{name}|{t.dtype}|{t.shape}|".encode())
            h.update(np.ascontiguousarray(flat[:n]).view(np.uint8).tobytes())
            h.update(np.ascontiguousarray(flat[-n:]).view(np.uint8).tobytes())
        return h.hexdigest()[:16]

    def named(self, fill: str = "read", seed: int = 0) -> dict[str, np.ndarray]:
        """The tensors by dotted name: ``"read"`` the file's (lazy views), ``"random"`` or
        ``"unread"`` ``filled``'s in the file's shapes, which reads nothing past the header."""
        if fill not in ("read", "random", "unread"):
            raise ValueError(f"fill is read, random or unread, not {fill!r}")
        if fill == "read":
            return dict(self.tensors)
        return filled(fill, {n: (t.shape, t.dtype) for n, t in self.tensors.items()}, seed)

    def tree(self, fill: str = "read", seed: int = 0):
        """The tensors as a tree split at the dots (lists where the names are indices)."""
        return nest(self.named(fill, seed), file=self.path)


# ---- trees ---------------------------------------------------------------------------------

_FILE = "the checkpoint"


class _Module(SimpleNamespace):
    """A module of a tree; a name it lacks raises an ``AttributeError`` that says where."""

    def __getattr__(self, name):
        if name.startswith("_"):
            raise AttributeError(name)
        have = ", ".join(k for k in vars(self) if not k.startswith("_")) or "nothing"
        raise AttributeError(f"{self._path}{name} is not in {self._file} (it has {have})")


class _Layers(list):
    """A run of modules by index; an index past the end raises an ``IndexError`` that says where."""

    def __getitem__(self, index):
        try:
            return super().__getitem__(index)
        except IndexError:
            raise IndexError(f"{self._path}{index} is not in {self._file} (it has {len(self)})") from None


def _build(node, path: str, file):
    if not isinstance(node, dict):
        return node
    built = {k: _build(v, f"{path}{k}.", file) for k, v in node.items()}
    if built and all(k.isdigit() for k in built):
        top = max(map(int, built))
        # a skipped index is a module without weights, never most of the run
        if top >= 4 * len(built) + 4:
            raise ValueError(f"{file}: {path}{top} is past its {len(built)} layers")
        out = _Layers(built[str(i)] if str(i) in built else _build({}, f"{path}{i}.", file) for i in range(top + 1))
    else:
        out = _Module(**built)
    out._path, out._file = path, file
    return out


def nest(named: Mapping[str, Any], path: str = "", file=_FILE):
    """Nest values by dotted name, under ``path`` (a dotted prefix) of ``file``."""
    root: dict = {}
    for name, value in named.items():
        *parents, leaf = name.split(".")
        node = root
        for key in parents:
            node = node.setdefault(key, {})
        node[leaf] = value
    return _build(root, path, file)


def leaves(tree, prefix: str = "") -> Iterator[tuple[str, Any]]:
    """Each leaf of a tree by its dotted name: ``nest``'s inverse."""
    if isinstance(tree, list):
        for i, v in enumerate(tree):
            yield from leaves(v, f"{prefix}{i}.")
    elif isinstance(tree, SimpleNamespace):
        for k, v in vars(tree).items():
            if not k.startswith("_"):
                yield from leaves(v, f"{prefix}{k}.")
    else:
        yield prefix[:-1], tree


def subtree(tree, **modules):
    """A tree of ``modules``, each a module of ``tree``, at their names (a text decoder out of a
    vision-language checkpoint)."""
    file = tree._file if isinstance(tree, (_Module, _Layers)) else _FILE
    return _build(dict(modules), "", file)


def renamed(tree, renames: Mapping[str, str]):
    """A copy of ``tree`` with each leaf under a run of whole dotted names moved to the run its
    value names; the rest stay."""

    def moved(path: str) -> str:
        for old, new in renames.items():
            at = f".{path}.".find(f".{old}.")
            if at >= 0:
                return path[:at] + new + path[at + len(old):]
        return path

    held = isinstance(tree, (_Module, _Layers))
    return nest({moved(p): v for p, v in leaves(tree)}, tree._path if held else "", tree._file if held else _FILE)


# ---- host to device --------------------------------------------------------------------------


class Uploader:
    """Copies host arrays into device tensors through a ring of pinned staging buffers.

    ``put(array, out)`` copies ``array`` (any float dtype, cast to ``out``'s) piecewise into
    the next free staging buffer and issues the host-to-device copy on a side stream; the
    host only waits when the ring wraps onto a buffer whose copy is still in flight.
    ``release`` (a ``Checkpoint.release``) is called on each array once its bytes are staged.
    """

    _pinned: dict = {}   # (slot_bytes, slots) -> staging buffers, pinned once per process

    def __init__(self, device="cuda", slot_bytes: int = 32 << 20, slots: int = 3, release=None):
        import torch

        self._torch = torch
        self.device = torch.device(device)
        self.release = release
        if self.device.type == "cuda":
            key = (slot_bytes, slots)
            if key not in Uploader._pinned:
                Uploader._pinned[key] = [torch.empty(slot_bytes, dtype=torch.uint8).pin_memory()
                                         for _ in range(slots)]
            self._slots = Uploader._pinned[key]
        else:
            self._slots = [torch.empty(slot_bytes, dtype=torch.uint8) for _ in range(slots)]
        self._done = [None] * slots
        self._at = 0
        self._stream = torch.cuda.Stream(self.device) if self.device.type == "cuda" else None
        self.bytes = 0

    def _stage(self, flat: np.ndarray, out_flat) -> None:
        torch = self._torch
        item = out_flat.element_size()
        per = self._slots[0].numel() // item
        np_out = {torch.bfloat16: bfloat16, torch.float32: np.float32, torch.float16: np.float16,
                  torch.int32: np.int32, torch.int64: np.int64}[out_flat.dtype]
        for lo in range(0, flat.size, per):
            hi = min(flat.size, lo + per)
            i = self._at
            self._at = (i + 1) % len(self._slots)
            if self._done[i] is not None:
                self._done[i].synchronize()
            host = self._slots[i][: (hi - lo) * item]
            piece = flat[lo:hi]
            np.copyto(host.numpy().view(np_out), piece if piece.dtype == np_out else piece.astype(np_out))
            if self._stream is None:
                out_flat[lo:hi].copy_(host.view(out_flat.dtype))
                continue
            with torch.cuda.stream(self._stream):
                out_flat[lo:hi].copy_(host.view(out_flat.dtype), non_blocking=True)
                ev = torch.cuda.Event()
                ev.record()
            self._done[i] = ev
            self.bytes += (hi - lo) * item

    def put(self, array, out) -> None:
        a = np.asarray(array)
        if a.size != out.numel():
            raise ValueError(f"{tuple(a.shape)} does not fill {tuple(out.shape)}")
        if not out.is_contiguous():
            # a strided destination (a row slice of a packed matrix) is filled row by row
            if a.ndim != 2 or out.dim() != 2 or not out[0].is_contiguous():
                raise ValueError("a strided destination is a run of contiguous rows")
            for r in range(a.shape[0]):
                self._stage(np.ascontiguousarray(a[r]).reshape(-1), out[r])
        else:
            src = a if a.flags.c_contiguous else np.ascontiguousarray(a)
            self._stage(src.reshape(-1), out.view(-1))
        if self.release is not None:
            self.release(a)

    def finish(self) -> None:
        """Wait for every copy issued so far: the tensors may then be read on any stream, and
        the staging buffers reused by another ``Uploader``."""
        if self._stream is not None:
            self._torch.cuda.current_stream(self.device).wait_stream(self._stream)
            self._stream.synchronize()
        self._done = [None] * len(self._slots)
