"""A device-side wait that runs out returns an error status and leaves the GPU usable (B200).

Every spin in the library's kernels has a wall-clock limit.  This test lets one of them run
out in the only way that needs no second process and faults nothing: the peer-memory
all-reduce is launched as rank 0 of a world of two whose second "rank" is a buffer on the
same GPU that nobody ever writes, so rank 1's flag is never raised.  The kernel gives up
after its limit, writes IRON_ERR_TIMEOUT to the status word, finishes with what it has and
returns; the context stays healthy and the next launch works.
"""

import ctypes
import time

import pytest

pytestmark = pytest.mark.gpu


def test_a_flag_nobody_raises_ends_in_a_timeout_status_not_a_hang():
    import torch

    from iron_b200 import kernels as K

    n = 2048
    nbytes = K.tp_buffer_bytes(2, n)
    mine = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")
    absent = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")   # the rank that never joins
    peers = (ctypes.c_void_p * 2)(mine.data_ptr(), absent.data_ptr())
    seq = torch.zeros(1, dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    part = torch.ones(n, dtype=torch.bfloat16, device="cuda")
    out = torch.empty_like(part)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    K.tp_allreduce(part, out, peer_buffers=peers, slot_elems=n, rank=0, world=2, seq=seq, status=status)
    torch.cuda.synchronize()
    waited = time.perf_counter() - t0
    assert int(status.item()) == -6                     # IRON_ERR_TIMEOUT, reported not raised
    assert 1.0 < waited < 10.0                          # it waited its limit, and only that
    assert int(seq.item()) == 1                         # the kernel ran to its end
    # rank 0's own partial arrived in both buffers; the absent rank's slot is still zero
    assert torch.equal(out, part)
    # the context is intact: the same call with every flag present completes at once
    status.zero_()
    # play rank 1 by hand for the second all-reduce (sequence 1, parity 1): its slot and flag in `mine`
    slots = mine[256 : 256 + 2 * 2 * n * 2].view(torch.bfloat16).view(2, 2, n)   # this kernel's bf16 slots
    slots[1, 1] = 2.0
    mine[:256].view(torch.int32)[1 * 2 + 1] = 2
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    K.tp_allreduce(part, out, peer_buffers=peers, slot_elems=n, rank=0, world=2, seq=seq, status=status)
    torch.cuda.synchronize()
    assert time.perf_counter() - t0 < 1.0
    assert int(status.item()) == 0
    assert torch.equal(out, torch.full_like(part, 3.0))
