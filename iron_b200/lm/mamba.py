"""A Mamba2 mixer as fused sm_100a kernels: what a compiled ``Mamba`` graph of the reference
becomes on B200 when throughput matters.

The reference records the mixer (iron/applications/granite_hybrid/model.py:120-137) as three
projections on row slices of ``in_proj``, the causal convolution as a chain of row-wise
products and sums (iron/functional.py:147-180) plus a bias add, SiLU, the scan
(iron/operators/selective_scan.py:46), SiLU of the gate, a product, RMSNorm over ``d_inner``
and ``out_proj``: about twenty steps.  Here a call of ``rows`` positions for ``batch``
independent sequences is seven launches:

    1-3. gate, x/B/C and dt projections              (iron_gemm_bf16, tcgen05)
    4.   causal convolution + bias + SiLU            (iron_causal_conv1d_bf16)
    5.   selective scan                              (iron_selective_scan_bf16)
    6.   RMSNorm over d_inner of y * silu(gate)      (iron_rmsnorm_gated_bf16)
    7.   out_proj                                    (iron_gemm_bf16)

with every rounding of the recorded steps kept (each projection, the convolution's chain, the
activation, the product and the norm's two roundings round to bf16 where the reference's
operators do), so the fused call and the recorded graph agree to the last bit wherever the
scan does.  The convolution's last ``kernel - 1`` rows and the scan's float32 state carry
from call to call, one set per sequence, as the reference's ``Checkpoints`` do
(iron/lm/causal.py:71-121).
"""

from __future__ import annotations

import numpy as np
import torch

from .. import kernels as K

BF16 = torch.bfloat16


def _device_bf16(a, device) -> torch.Tensor:
    if isinstance(a, torch.Tensor):
        return a.to(device=device, dtype=BF16).contiguous()
    a = np.ascontiguousarray(a)
    if a.dtype.name == "bfloat16":
        return torch.from_numpy(a.view(np.int16)).view(BF16).to(device)
    return torch.from_numpy(a.astype(np.float32)).to(device).to(BF16)


class MambaMixer:
    """One mixer on ``weights`` (the checkpoint's names under ``prefix``: ``in_proj.weight``,
    ``conv1d.weight``, ``conv1d.bias``, ``dt_bias``, ``A_log``, ``D``, ``norm.weight``,
    ``out_proj.weight``) for calls of up to ``rows`` positions of ``batch`` sequences."""

    def __init__(self, weights: dict, *, hidden_size: int, heads: int, head_dim: int, state_size: int,
                 groups: int = 1, kernel: int = 4, eps: float = 1e-5, batch: int = 1, rows: int = 2048,
                 prefix: str = "", device="cuda"):
        if not torch.cuda.is_available():
            raise RuntimeError("MambaMixer needs a CUDA device: there is no CPU path")
        self.device = torch.device(device)
        self.E, self.H, self.P, self.N, self.G, self.Kc = hidden_size, heads, head_dim, state_size, groups, kernel
        self.inner = heads * head_dim
        self.channels = self.inner + 2 * groups * state_size
        self.eps, self.batch, self.rows = eps, batch, rows
        w = lambda n: weights[prefix + n]
        dev = self.device
        in_proj = _device_bf16(w("in_proj.weight"), dev)
        if tuple(in_proj.shape) != (self.inner + self.channels + heads, hidden_size):
            raise ValueError(f"in_proj.weight is {tuple(in_proj.shape)}, the mixer's shape asks "
                             f"{(self.inner + self.channels + heads, hidden_size)}")
        # the three projections read row slices of the one matrix in place
        self.w_gate = in_proj[: self.inner]
        self.w_xbc = in_proj[self.inner : self.inner + self.channels]
        self.w_dt = in_proj[self.inner + self.channels :]
        conv = _device_bf16(w("conv1d.weight"), dev).reshape(self.channels, kernel)
        self.taps = conv.t().contiguous()                       # one row per tap
        self.conv_bias = _device_bf16(w("conv1d.bias"), dev)
        f32 = lambda a: torch.as_tensor(np.asarray(a, np.float32) if not isinstance(a, torch.Tensor)
                                        else a.float().cpu().numpy())
        A = -torch.exp(f32(w("A_log")))
        self.head = torch.stack([f32(w("dt_bias")), A, f32(w("D"))], 1).contiguous().to(dev)   # (H, 3) f32
        self.norm_w = _device_bf16(w("norm.weight"), dev)
        self.w_out = _device_bf16(w("out_proj.weight"), dev)
        n = batch * rows
        new = lambda *shape, dtype=BF16: torch.empty(shape, dtype=dtype, device=dev)
        self.gate, self.xbc, self.dt = new(n, self.inner), new(n, self.channels), new(n, heads)
        self.conv_out, self.y, self.out = new(n, self.channels), new(n, self.inner), new(n, hidden_size)
        self.normed = new(n, self.inner)
        self.conv_state = torch.zeros(batch, kernel - 1, self.channels, dtype=BF16, device=dev)
        self.ssm_state = torch.zeros(batch, heads, head_dim, state_size, dtype=torch.float32, device=dev)
        self.status = torch.zeros(1, dtype=torch.int32, device=dev)

    launches_per_call = 7

    def reset(self) -> None:
        """Forget every sequence: zero convolution rows and scan states."""
        self.conv_state.zero_()
        self.ssm_state.zero_()

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        """``x`` (batch, rows, hidden) bf16 -> (batch, rows, hidden) bf16, the states advanced.

        ``rows`` may be anything up to the mixer's; one row is a decode step (the convolution
        then sums its taps in the decode step's order, iron/functional.py:165-167)."""
        if x.dim() != 3 or x.shape[0] != self.batch or x.shape[2] != self.E or not 0 < x.shape[1] <= self.rows:
            raise ValueError(f"x is {tuple(x.shape)}; the mixer takes ({self.batch}, 1..{self.rows}, {self.E})")
        B, R = x.shape[0], x.shape[1]
        n = B * R
        x2 = x.reshape(n, self.E)
        gate, xbc, dt = self.gate[:n], self.xbc[:n], self.dt[:n]
        K.gemm(x2, self.w_gate, gate, b_col_maj=True, status=self.status)
        K.gemm(x2, self.w_xbc, xbc, b_col_maj=True, status=self.status)
        K.gemm(x2, self.w_dt, dt, b_col_maj=True, status=self.status)
        conv = self.conv_out[:n].view(B, R, self.channels)
        K.causal_conv1d(xbc.view(B, R, self.channels), self.taps, bias=self.conv_bias, history=self.conv_state,
                        new_history=self.conv_state, out=conv, decode_order=(R == 1), silu=True)
        y = self.y[:n].view(B, R, self.inner)
        K.selective_scan(conv, dt.view(B, R, self.H), self.head, self.ssm_state, heads=self.H, head_dim=self.P,
                         state_size=self.N, groups=self.G, y=y, final=self.ssm_state)
        K.rms_norm_gated(self.y[:n], gate, self.norm_w, self.normed[:n], eps=self.eps)
        out = self.out[:n]
        K.gemm(self.normed[:n], self.w_out, out, b_col_maj=True, status=self.status)
        return out.view(B, R, self.E)

    def check(self) -> None:
        if int(self.status.item()) != 0:
            raise RuntimeError("a GEMM pipeline wait gave up (IRON_ERR_TIMEOUT)")
