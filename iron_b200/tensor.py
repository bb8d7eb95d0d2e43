"""The host-visible tensor a standalone operator call takes.

The reference's ``aie.utils.DEFAULT_TENSOR_CLASS`` (iron/common/testing.py:163-169,
:268-282): ``Tensor(np_array)`` or ``Tensor(shape, dtype=)``, ``.numpy()`` to read back and
``.data`` for a host view.  Here the storage is a CUDA tensor (``.torch``).
"""

from __future__ import annotations

import contextlib
import gc

import numpy as np
from ml_dtypes import bfloat16


def _torch():
    import torch

    if not torch.cuda.is_available():
        raise RuntimeError("iron_b200 tensors live on a CUDA device; none is available")
    return torch


@contextlib.contextmanager
def capturing(graph, **kw):
    """``torch.cuda.graph`` with the garbage collector held off.

    A collection that runs while a stream is capturing may free an older ``CUDAGraph``; its
    teardown is a call the capture does not allow and invalidates it.  So collect first,
    then keep the collector off until the capture has ended.
    """
    torch = _torch()
    was = gc.isenabled()
    gc.collect()
    gc.disable()
    try:
        with torch.cuda.graph(graph, **kw):
            yield graph
    finally:
        if was:
            gc.enable()


def numpy_to_torch(a: np.ndarray, device="cuda"):
    torch = _torch()
    a = np.ascontiguousarray(a)
    if a.dtype == bfloat16:
        return torch.from_numpy(a.view(np.int16)).view(torch.bfloat16).to(device)
    return torch.from_numpy(a).to(device)


def torch_to_numpy(t) -> np.ndarray:
    torch = _torch()
    t = t.detach().cpu().contiguous()
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy().view(bfloat16)
    return t.numpy()


_TORCH_DTYPES = {"bfloat16": "bfloat16", "float32": "float32", "int32": "int32", "int64": "int64",
                 "float16": "float16", "uint8": "uint8", "int8": "int8", "int16": "int16"}


class Tensor:
    """A device buffer with a numpy face."""

    def __init__(self, array_or_shape, dtype=bfloat16, device="cuda"):
        torch = _torch()
        if isinstance(array_or_shape, np.ndarray):
            self.torch = numpy_to_torch(array_or_shape, device)
        elif isinstance(array_or_shape, torch.Tensor):
            self.torch = array_or_shape if array_or_shape.is_cuda else array_or_shape.to(device)
        else:
            name = _TORCH_DTYPES[np.dtype(dtype).name]
            self.torch = torch.zeros(tuple(array_or_shape), dtype=getattr(torch, name), device=device)

    @property
    def shape(self):
        return tuple(self.torch.shape)

    @property
    def dtype(self):
        return self.numpy().dtype

    def numpy(self) -> np.ndarray:
        return torch_to_numpy(self.torch)

    @property
    def data(self) -> np.ndarray:
        return self.numpy()

    def __repr__(self):
        return f"Tensor{self.shape}"


DEFAULT_TENSOR_CLASS = Tensor


def as_device(t) -> Tensor:
    """``t`` as a ``Tensor`` (numpy arrays are uploaded, torch CUDA tensors wrapped)."""
    return t if isinstance(t, Tensor) else Tensor(t)
