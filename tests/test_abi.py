"""The C-ABI library loads and exports every symbol include/iron_b200.h declares (no GPU)."""

import ctypes

from iron_b200 import _lib


def test_every_declared_symbol_is_exported_and_bound():
    lib = _lib.load()
    declared = _lib.declared_symbols()
    assert declared, "the header declares nothing?"
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared in include/iron_b200.h but not exported"
    assert set(declared) == set(_lib.SIGNATURES), (
        sorted(set(declared) ^ set(_lib.SIGNATURES)))


def test_version_and_arch():
    lib = _lib.load()
    assert lib.iron_version() >= 100
    assert lib.iron_arch() == b"sm_100a"


def test_bad_shapes_are_refused_before_any_launch():
    lib = _lib.load()
    # K not a multiple of 8; null pointers are never dereferenced on the host
    assert lib.iron_gemv_bf16(None, None, None, 16, 12, 1, 1, 16, 0, None, 1e-5, None, None) == -1
    assert lib.iron_rope_bf16(None, None, None, 4, 24, 4, 1, 0, None, 4, None, None) == -1
    assert lib.iron_mha_decode_bf16(None, None, None, None, 1, 6, 4, 64, 8, 0, 256, 64, 8, None, 0, 0,
                                    -1, 0.125, 1, 0, None) == -1
    assert lib.iron_mha_decode_splits(1, 8, 2048) == 8
    assert lib.iron_gemm_bf16(None, None, None, 0, 8, 8, 8, 8, 8, 1, 0, 0, None, 8, 0, None, 0, None,
                              None) == -1
