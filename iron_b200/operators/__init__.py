"""The operator library: one class per operator, and the catalogue the harness walks.

``CATALOG`` mirrors ``iron/operators/__init__.py:69-72`` for the operators on the decoder
and Mamba2 paths and the element-wise and row-wise operators beside them.
"""

from .axpy import AXPY
from .causal_conv import CausalConv1d
from .clamp import Clamp
from .copy import Copy, Gather
from .elementwise_add import ElementwiseAdd, RowwiseAdd
from .elementwise_mul import ElementwiseMul, RowwiseMul
from .flm.gemm.design import Epilogue
from .flm.gemm.op import ProjectionGEMM
from .gemm import GEMM
from .gelu import GELU
from .gemv import GEMV
from .layer_norm import LayerNorm
from .mha import MHA
from .relu import ReLU
from .rms_norm import RMSNorm
from .rope import RoPE
from .sample import Sample
from .selective_scan import SelectiveScan
from .sigmoid import Sigmoid
from .silu import SiLU
from .softmax import Softmax
from .tanh import Tanh

CATALOG = (GEMM, ProjectionGEMM, GEMV, RMSNorm, LayerNorm, RoPE, SiLU, Sigmoid, ReLU, Tanh, GELU, Clamp,
           ElementwiseAdd, RowwiseAdd, ElementwiseMul, RowwiseMul, AXPY, MHA, Softmax, Copy, Gather,
           SelectiveScan, CausalConv1d, Sample)

__all__ = [c.__name__ for c in CATALOG] + ["CATALOG", "Epilogue"]
