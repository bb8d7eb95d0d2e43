"""The workspace-free greedy draw, called through the C ABI.

`iron_argmax_bf16_noalloc` serves callers that cannot allocate device memory (a thread kept
out of the CUDA allocator, a plugin in a runtime that owns all device memory): its scratch
is a fixed array inside the library.  It must give exactly what `iron_argmax_bf16` gives with
a caller-provided workspace, on consecutive calls that reuse the array, and refuse more
logits than it is stated for.  This file sorts last so that a run stopping at the first
failure has already run every other test.
"""

import ctypes

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_no_alloc_argmax_matches_the_workspace_entry_point_twice_in_a_row():
    import torch

    from iron_b200 import _lib

    lib = _lib.load()
    stream = torch.cuda.current_stream().cuda_stream
    ws = torch.zeros(lib.iron_argmax_workspace_bytes(0), dtype=torch.uint8, device="cuda")
    for call, n in enumerate((128256, 1000)):   # two calls in a row share the built-in scratch
        gen = torch.Generator(device="cuda").manual_seed(100 + call)
        logits = (torch.randn(n, generator=gen, device="cuda") * 3).to(torch.bfloat16)
        top = logits.float().max()
        logits[n // 3] = top
        logits[n // 2] = top                     # a tie: the first index must win in both
        want = torch.full((4,), -1, dtype=torch.int32, device="cuda")
        got = torch.full((4,), -1, dtype=torch.int32, device="cuda")
        index = torch.tensor([2], dtype=torch.int32, device="cuda")
        carry_a = torch.tensor([0, 7], dtype=torch.int32, device="cuda")
        carry_b = torch.tensor([0, 7], dtype=torch.int32, device="cuda")
        rc = lib.iron_argmax_bf16(logits.data_ptr(), n, want.data_ptr(), index.data_ptr(), want.numel(),
                                  carry_a.data_ptr(), carry_a[1:].data_ptr(), ws.data_ptr(), stream)
        assert rc == 0
        rc = lib.iron_argmax_bf16_noalloc(logits.data_ptr(), n, got.data_ptr(), index.data_ptr(),
                                          carry_b.data_ptr(), carry_b[1:].data_ptr(), stream)
        assert rc == 0
        torch.cuda.synchronize()
        assert torch.equal(got, want), (got.tolist(), want.tolist())
        assert torch.equal(carry_a, carry_b) and carry_b.tolist()[1] == 8
        assert int(got[2]) == int(torch.argmax(logits.float()))  # first index of the maximum


def test_no_alloc_argmax_refuses_more_than_its_stated_maximum():
    import torch

    from iron_b200 import _lib

    lib = _lib.load()
    limit = lib.iron_argmax_noalloc_max_n()
    assert limit == 1 << 22
    small = torch.zeros(16, dtype=torch.bfloat16, device="cuda")
    out = torch.zeros(1, dtype=torch.int32, device="cuda")
    rc = lib.iron_argmax_bf16_noalloc(small.data_ptr(), limit + 1, out.data_ptr(), None, None, None, None)
    assert rc == -5   # IRON_ERR_WORKSPACE: refused on the host, nothing launched
    assert lib.iron_argmax_bf16_noalloc(small.data_ptr(), 0, out.data_ptr(), None, None, None, None) == -1
