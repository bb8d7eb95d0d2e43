"""ProjectionGEMM (iron/operators/flm/gemm/op.py:128): what ``F.linear`` records for several rows."""

import numpy as np

from ....declare import In, Operator, Out, Select, param, per_call, tunable
from ....lm.config import Precision
from ....testing import Case, Testing
from ....verify import Tolerance
from .design import Epilogue


def _cases(cls, dev=None):
    return [Case(dict(M=2048, K=2048, N=512, b_col_maj=True, precision=Precision.MEDIUM)),
            Case(dict(M=512, K=2048, N=2048, b_col_maj=True, precision=Precision.MEDIUM), bench=True),
            Case(dict(M=256, K=512, N=768, b_col_maj=True, precision=Precision.HIGH,
                      epilogue_modes=(Epilogue.SILU,)))]


class ProjectionGEMM(Operator):
    """``C = epilogue(bf16(A @ B))`` with the weight as the checkpoint stores it."""

    test = Testing(_cases, draw=lambda op: dict(normal=(op.A, op.B)))

    M: int = param()
    K: int = param()
    N: int = param()
    b_col_maj: bool = param(default=True, array=True)
    epilogue_modes: tuple = param(default=(Epilogue.NONE,), array=True)
    precision: Precision = param(default=Precision.MEDIUM, array=True)
    tile_n: int = tunable()
    num_aie_columns: int = tunable()

    A = In(M, K)
    B = In(Select(b_col_maj, (N, K), (K, N)))
    C = Out(M, N)
    valid = per_call(bounds=M)

    @property
    def epilogue(self) -> Epilogue:
        return Epilogue(self.epilogue_modes[0])

    def validate(self):
        if len(self.epilogue_modes) != 1:
            raise ValueError("ProjectionGEMM: one epilogue mode per operator here")
        if self.K % 8 or (not self.b_col_maj and self.N % 8):
            raise ValueError("ProjectionGEMM: row pitches must be multiples of 8 elements")

    def ops(self) -> int:
        return 2 * self.M * self.K * self.N

    def reference(self, A, B):
        b = B.T if self.b_col_maj else B
        C = np.matmul(A.astype(np.float32), b.astype(np.float32)).astype(A.dtype)
        return np.asarray(self.epilogue.apply(C)).astype(A.dtype)

    def tolerance(self):
        if self.epilogue is not Epilogue.NONE:
            return None
        units = 2.0 + self.K * 2.0 ** -16

        def bound(A, B):
            b = B.T if self.b_col_maj else B
            return units * 2.0 ** -8 * (np.abs(A.astype(np.float32)) @ np.abs(b.astype(np.float32)))

        return Tolerance.bounded(bound, note=f"{units:g} units of |A| @ |B|")

    def launch(self, buffers, values):
        from .... import kernels as K

        K.gemm(buffers["A"], buffers["B"], buffers["C"], b_col_maj=self.b_col_maj, valid=self.valid,
               epilogue=self.epilogue.value)
