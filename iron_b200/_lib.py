"""ctypes binding of ``libiron_b200.so`` (the C ABI declared in ``include/iron_b200.h``).

There is no CPU fallback: a missing library, or a call with no CUDA device, raises.
"""

from __future__ import annotations

import ctypes
import re
from ctypes import c_char_p, c_float, c_int, c_longlong, c_size_t, c_void_p
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "csrc" / "libiron_b200.so"
HEADER = Path(__file__).resolve().parents[1] / "include" / "iron_b200.h"

ERRORS = {
    0: "ok",
    -1: "IRON_ERR_SHAPE: a size the kernel family refuses",
    -2: "IRON_ERR_ALIGN: a pointer or pitch is not 16-byte aligned",
    -3: "IRON_ERR_LAUNCH: the CUDA runtime reported a launch error",
    -4: "IRON_ERR_UNSUPPORTED: a mode this build does not implement",
    -5: "IRON_ERR_WORKSPACE: the workspace given is too small",
    -6: "IRON_ERR_TIMEOUT: a bounded device-side wait gave up",
}


class IronError(RuntimeError):
    """A C-ABI entry point returned a negative status."""

    def __init__(self, name: str, code: int):
        self.code = code
        super().__init__(f"{name} failed: {ERRORS.get(code, code)}")


_P, _I, _L, _F, _Z = c_void_p, c_int, c_longlong, c_float, c_size_t

# name -> (restype, argtypes).  Kept in step with include/iron_b200.h; the CPU test
# suite checks that the two agree symbol by symbol.
SIGNATURES: dict[str, tuple] = {
    "iron_version": (_I, []),
    "iron_arch": (c_char_p, []),
    "iron_set_pdl": (None, [_I]),
    "iron_prefetch_hint": (_I, [_P, _L]),
    "iron_gemv_bf16": (_I, [_P, _P, _P, _I, _I, _I, _I, _I, _I, _P, _F, _P, _P]),
    "iron_gemv_swiglu_bf16": (_I, [_P, _P, _P, _P, _I, _I, _I, _P, _F, _P]),
    "iron_decode_qkv_rope_bf16": (
        _I,
        [_P, _P, _I, _I, _P, _F, _P, _I, _P, _P, _P, _P, _I, _I, _I, _I, _P],
    ),
    "iron_decode_attn_oproj_scratch_bytes": (_Z, [_I, _I]),
    "iron_decode_attn_oproj_supported": (_I, [_I, _I, _I, _I]),
    "iron_decode_attn_oproj_trace": (None, [_P]),
    "iron_decode_attn_oproj_bf16": (
        _I,
        [_P, _P, _P, _I, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _F, _P, _P, _P],
    ),
    "iron_gemm_bf16": (
        _I,
        [_P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _I, _P, _I, _I, _P, _I, _P, _P],
    ),
    "iron_gemm_swiglu_bf16": (_I, [_P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _P, _P, _P]),
    "iron_rmsnorm_bf16": (_I, [_P, _P, _P, _I, _I, _F, _I, _P, _P]),
    "iron_rmsnorm_gated_bf16": (_I, [_P, _P, _P, _P, _I, _I, _F, _I, _P, _P]),
    "iron_rope_bf16": (_I, [_P, _P, _P, _I, _I, _I, _I, _I, _P, _I, _P, _P]),
    "iron_rope_kv_write_bf16": (_I, [_P, _L, _P, _P, _P, _I, _P, _I, _I, _I, _I, _P, _I, _P, _P]),
    "iron_elementwise_bf16": (_I, [_I, _P, _P, _P, _L, _I, _F, _P]),
    "iron_softmax_bf16": (_I, [_P, _I, _P, _P, _I, _I, _I, _P, _F, _P]),
    "iron_clamp_bf16": (_I, [_P, _P, _L, _F, _F, _P]),
    "iron_layernorm_bf16": (_I, [_P, _P, _P, _I, _I, _F, _I, _P, _P]),
    "iron_copy_rows": (_I, [_P, _P, _P, _I, _P, _L, _L, _L, _I, _I, _P, _I, _P, _P]),
    "iron_argmax_workspace_bytes": (_Z, [_I]),
    "iron_argmax_bf16": (_I, [_P, _I, _P, _P, _I, _P, _P, _P, _P]),
    "iron_argmax_key_bf16": (_I, [_P, _I, _I, _P, _P, _P]),
    "iron_argmax_pick": (_I, [_P, _I, _P, _P, _I, _P, _P, _P]),
    "iron_argmax_noalloc_max_n": (_I, []),
    "iron_argmax_bf16_noalloc": (_I, [_P, _I, _P, _P, _P, _P, _P]),
    "iron_tp_buffer_bytes": (_Z, [_I, _I]),
    "iron_tp_allreduce_bf16": (_I, [_P, _P, _P, _I, _I, _P, _I, _I, _P, _P, _P]),
    "iron_tp_allreduce_tagged_bf16": (_I, [_P, _P, _P, _I, _I, _P, _I, _I, _P, _P, _P]),
    "iron_tp_push_next": (_I, [_P, _I, _I, _I, _P, _P]),
    "iron_tp_pull_next": (_I, [_P, _I, _I, _I, _P, _P, _P, _P]),
    "iron_gemm_rows_parts": (_I, [_I, _I, _I, _I]),
    "iron_gemm_rows_bf16": (_I, [_P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _P, _P, _I, _F, _P, _P, _P]),
    "iron_gemm_rows_qkv_rope_bf16": (
        _I,
        [_P, _P, _I, _I, _I, _I, _P, _P, _I, _F, _P, _P, _P, _P, _P, _L, _I, _I, _I, _I, _P, _P],
    ),
    "iron_rope_kv_scatter_bf16": (_I, [_P, _L, _P, _P, _P, _P, _L, _I, _P, _I, _I, _I, _I, _P]),
    "iron_argmax_rows_bf16": (_I, [_P, _L, _I, _I, _P, _P, _P, _I, _P]),
    "iron_decode_step_workspace_bytes": (_Z, [_I, _I, _I, _I]),
    "iron_decode_step_maps_bytes": (_Z, [_I]),
    "iron_decode_step_encode_maps": (_I, [_P, _I, _I, _I, _I, _I, _I, _I, _P, _P]),
    "iron_decode_step_bf16": (
        _I,
        [_P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _P, _P, _P, _P, _F, _F, _I, _P, _P, _P, _P, _P, _P, _P, _P],
    ),
    "iron_mha_decode_splits": (_I, [_I, _I, _I]),
    "iron_mha_decode_bf16": (
        _I,
        [_P, _P, _P, _P, _I, _I, _I, _I, _I, _L, _L, _L, _I, _P, _I, _I, _I, _F, _I, _I, _P],
    ),
    "iron_set_scan_chunked": (None, [_I]),
    "iron_selective_scan_status_word": (None, [_P]),
    "iron_selective_scan_bf16": (_I, [_P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _P, _P]),
    "iron_causal_conv1d_bf16": (_I, [_P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _P, _I, _I, _P]),
    "iron_gemm_qkv_rope_bf16": (_I, [_P, _P, _P, _I, _I, _I, _I, _I, _I, _P, _P, _P, _I, _I, _I, _I, _I, _P, _P]),
    "iron_sample_k_max": (_I, []),
    "iron_sample_rows_bf16": (_I, [_P, _L, _I, _I, _P, _P, _P, _P, _I, _P]),
    "iron_mha_prefill_status_word": (None, [_P]),
    "iron_mha_prefill_bf16": (
        _I,
        [_P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _L, _L, _L, _L, _L, _L, _L, _L, _L, _I, _P, _I, _P, _I, _I, _I, _F, _P],
    ),
}

_lib = None


def declared_symbols() -> list[str]:
    """Every function ``include/iron_b200.h`` declares."""
    text = HEADER.read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(iron_[a-z0-9_]+)\s*\(", text)))


def load() -> ctypes.CDLL:
    """Load the shared library (once) and attach argument types."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m iron_b200.build` "
            "(there is no CPU fallback)"
        )
    lib = ctypes.CDLL(str(LIB_PATH))
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = res, args
    _lib = lib
    return lib


def call(name: str, *args):
    """Call a status-returning entry point; raise ``IronError`` on a negative status."""
    rc = getattr(load(), name)(*args)
    if rc != 0:
        raise IronError(name, rc)
