"""GEMV (iron/operators/gemv.py:79)."""

import numpy as np

from ..declare import In, Operator, Out, param, per_call, tunable
from ..testing import Case, Testing
from ..verify import Tolerance


def _cases(cls, dev=None):
    # the reference's plain, batched and repeated shapes (iron/operators/gemv.py:24-76)
    plain = [(128, 128), (2048, 8192), (8192, 2048), (1536, 12288)]
    batched = [(256, 128, 4), (256, 128, 100), (448, 64, 192), (64, 1536, 8), (1026, 64, 2),
               (1024, 1024, 2), (512, 64, 32)]
    repeated = [(256, 128, 8, 4), (256, 128, 4, 4), (1024, 1024, 4, 2), (2048, 64, 32, 4)]
    return ([Case(dict(M=m, K=k), bench=m * k >= 2048 * 8192) for m, k in plain]
            + [Case(dict(M=m, K=k, num_batches=b)) for m, k, b in batched]
            + [Case(dict(M=m, K=k, num_batches=b, repeat=r)) for m, k, b, r in repeated])


class GEMV(Operator):
    """``C = A @ B`` for one vector (or one per batch); float32 accumulation, one rounding."""

    test = Testing(_cases, draw=lambda op: dict(normal=(op.A, op.B)))

    M: int = param()
    K: int = param()
    num_batches: int | None = param(default=None)
    repeat: int = param(default=1)
    num_matrices: int | None = param(
        derive=lambda op: None if op.num_batches is None else op.num_batches // op.repeat)
    num_aie_columns: int = tunable()
    num_channels: int = tunable()
    tile_size_input: int = tunable()
    tile_size_output: int = tunable()
    kernel_vector_size: int = tunable(repr=False)

    A = In(num_matrices, M, K)
    B = In(num_batches, K)
    C = Out(num_batches, M)
    valid = per_call(bounds=M)

    def validate(self):
        if self.K % 8:
            raise ValueError(f"GEMV: K ({self.K}) must be a multiple of 8")
        if self.num_batches is not None and self.num_batches % self.repeat:
            raise ValueError(f"GEMV: repeat ({self.repeat}) must divide num_batches ({self.num_batches})")

    def ops(self) -> int:
        return 2 * self.M * self.K * (self.num_batches or 1)

    def reference(self, A, B):
        if self.repeat > 1:
            A = np.repeat(A.reshape(-1, *A.shape[-2:]), self.repeat, axis=0)
        a, b = A.astype(np.float32), B.astype(np.float32)
        if A.ndim == 3:
            b = b.reshape(A.shape[0], A.shape[2], 1)
            return np.matmul(a, b).reshape(A.shape[0], A.shape[1]).astype(A.dtype)
        return (a @ b.reshape(A.shape[-1])).astype(A.dtype)

    def tolerance(self) -> Tolerance:
        return Tolerance.relative(0.04, 1e-3, note="f32 accumulation, rounded once")

    def launch(self, buffers, values):
        from .. import kernels as K

        K.gemv(buffers["A"], buffers["B"], buffers["C"], repeat=self.repeat, valid=self.valid)
