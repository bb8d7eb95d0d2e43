"""GEMM (iron/operators/gemm.py:143) on the tcgen05 tensor cores."""

from typing import Any

import numpy as np
from ml_dtypes import bfloat16

from ..declare import In, Operator, Out, Select, param, per_call, tunable
from ..lm.config import Precision
from ..testing import Case, Testing
from ..verify import Tolerance


def _cases(cls, dev=None):
    shapes = [(64, 64, 64), (256, 256, 256), (2048, 2048, 2048), (2048, 512, 2048), (384, 1536, 768)]
    out = [Case(dict(M=m, K=k, N=n, precision=Precision.HIGHEST), bench=m * k * n >= 2 ** 33) for m, n, k in shapes]
    out += [Case(dict(M=512, K=256, N=384, precision=Precision.HIGHEST, b_col_maj=True)),
            Case(dict(M=512, K=256, N=384, precision=Precision.HIGHEST, c_col_maj=True)),
            Case(dict(M=256, K=256, N=256, precision=Precision.HIGHEST, output_dtype=np.float32))]
    return out


class GEMM(Operator):
    """``C = A @ B``; bf16 in, float32 accumulation in tensor memory, one rounding."""

    test = Testing(_cases, draw=lambda op: dict(normal=(op.A,)))

    M: int = param()
    K: int = param()
    N: int = param()
    tile_m: int = tunable()
    tile_k: int = tunable(default=64)
    tile_n: int = tunable(default=64)
    num_aie_columns: int = tunable()
    placement: Any = tunable()
    b_col_maj: bool = param(default=False, array=True)
    c_col_maj: bool = param(default=False, array=True)
    precision: Precision = param(default=Precision.HIGHEST, array=True)
    accumulate_f32: bool = param(default=False, array=True)
    input_dtype: Any = param(default=bfloat16, repr=False)
    output_dtype: Any = param(default=bfloat16, repr=False)

    A = In(M, K, dtype=input_dtype)
    B = In(Select(b_col_maj, (N, K), (K, N)), dtype=input_dtype)
    C = Out(Select(c_col_maj, (N, M), (M, N)), dtype=output_dtype)
    valid = per_call(bounds=M)
    valid_k = per_call(bounds=K)

    def validate(self):
        if np.dtype(self.input_dtype) != np.dtype(bfloat16):
            raise ValueError("GEMM: inputs are bfloat16 on this device")
        if np.dtype(self.output_dtype) not in (np.dtype(bfloat16), np.dtype(np.float32)):
            raise ValueError("GEMM: the output is bfloat16 or float32")
        if self.K % 8 or (not self.b_col_maj and self.N % 8):
            raise ValueError("GEMM: row pitches must be multiples of 8 elements")

    def ops(self) -> int:
        return 2 * self.M * self.K * self.N

    def reference(self, A, B):
        a = A.astype(np.float32)[:, : self.valid_k]
        b = (B.T if self.b_col_maj else B).astype(np.float32)[: self.valid_k]
        C = np.matmul(b.T, a.T) if self.c_col_maj else np.matmul(a, b)
        return C.astype(self.output_dtype)

    def tolerance(self) -> Tolerance:
        # every precision level runs bf16 x bf16 with float32 partial sums here: 2 units
        def bound(A, B):
            a = A.astype(np.float32)
            b = (B.T if self.b_col_maj else B).astype(np.float32)
            err = 2.0 * (np.abs(a) @ np.abs(b)) * 2.0 ** -8
            return err.T if self.c_col_maj else err

        return Tolerance.bounded(bound, note="2 units of |A| @ |B|")

    def launch(self, buffers, values):
        from .. import kernels as K

        K.gemm(buffers["A"], buffers["B"], buffers["C"], b_col_maj=self.b_col_maj, c_col_maj=self.c_col_maj,
               valid=self.valid, valid_k=self.valid_k,
               out_f32=np.dtype(self.output_dtype) == np.dtype(np.float32))
