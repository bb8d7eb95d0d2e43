"""Copy and Gather (iron/operators/copy.py:546, :72): exact data movement.

The reference's ``Copy`` moves between arbitrary access patterns with per-call offsets; a
graph's handles lower indexing and slice assignment to it.  Here a ``Copy`` moves ``rows``
rows of ``cols`` elements between two row-strided views, each with an optional per-call
first row, and a ``Gather`` picks rows of a table by (clipped) ids -- the forms the decoder
path records (embedding rows, KV-cache rows, RoPE rows, the last prompt row).
"""

import numpy as np
from ml_dtypes import bfloat16

from ..declare import In, Operator, Out, param, per_call
from ..testing import Case, Testing
from ..verify import Tolerance


class Copy(Operator):
    """``dst[dst_row + i] = src[src_row + i]`` for ``i < valid``."""

    test = Testing([Case(dict(rows=16, cols=512, src_rows=64, dst_rows=64)),
                    Case(dict(rows=2048, cols=512, src_rows=2048, dst_rows=4096), bench=True)])

    rows: int = param()
    cols: int = param()
    src_rows: int = param(default=lambda op: op.rows)
    dst_rows: int = param(default=lambda op: op.rows)
    dtype: object = param(default=bfloat16, repr=False)

    src = In(src_rows, cols, dtype=dtype)
    dst = Out(dst_rows, cols, dtype=dtype)
    valid = per_call(bounds=rows)
    src_row = per_call()
    dst_row = per_call()

    def __getattr__(self, name):
        if name in ("src_row", "dst_row"):
            return self.__dict__.get("bound_extents", {}).get(name, 0)
        return super().__getattr__(name)

    def validate(self):
        if (self.cols * np.dtype(self.dtype).itemsize) % 16:
            raise ValueError("Copy: a row must be a multiple of 16 bytes")

    def ops(self) -> int:
        return 0

    def reference(self, src):
        out = np.zeros((self.dst_rows, self.cols), src.dtype)
        out[self.dst_row : self.dst_row + self.valid] = src[self.src_row : self.src_row + self.valid]
        return out

    def tolerance(self):
        return Tolerance.exact(note="data movement")

    def launch(self, buffers, values):
        from .. import kernels as K

        nbytes = self.cols * np.dtype(self.dtype).itemsize
        K.copy_rows(buffers["src"], buffers["dst"], nrows=self.valid, row_bytes=nbytes,
                    src_row0=self.src_row, dst_row0=self.dst_row, d_nrows=values.get("d_valid"),
                    d_src_row0=values.get("d_src_row"), d_dst_row0=values.get("d_dst_row"))


class Gather(Operator):
    """``out[i] = table[clip(ids[i])]``: embedding rows."""

    test = Testing([Case(dict(rows=8, cols=2048, table_rows=1024)),
                    Case(dict(rows=2048, cols=2048, table_rows=128256), bench=True)],
                   draw=lambda op: dict(given={op.ids: np.random.default_rng(1).integers(
                       -2, op.table_rows + 2, op.rows).astype(np.int32)}))

    rows: int = param()
    cols: int = param()
    table_rows: int = param()

    table = In(table_rows, cols)
    ids = In(rows, dtype=np.int32)
    out = Out(rows, cols)
    valid = per_call(bounds=rows)

    def ops(self) -> int:
        return 0

    def reference(self, table, ids):
        picked = table[np.clip(ids.astype(np.int64), 0, self.table_rows - 1)]
        picked[self.valid:] = 0
        return picked

    def tolerance(self):
        return Tolerance.exact(note="data movement")

    def launch(self, buffers, values):
        from .. import kernels as K

        K.copy_rows(buffers["table"], buffers["out"], ids=buffers["ids"], nrows=self.valid,
                    row_bytes=self.cols * 2, src_rows=self.table_rows, d_nrows=values.get("d_valid"))
