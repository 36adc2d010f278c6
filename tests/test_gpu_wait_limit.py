"""GPU: a bounded device-side wait that runs out.  scmx_peer_barrier is called for a world of two ranks on two local flag
arrays that nobody else signals, with the wait limit lowered to 2 ms: the kernel must return by itself, leave code 20 in the
status word, and check_status() must raise.  Nothing faults, traps or spins without a limit."""
import ctypes
import time

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_peer_barrier_wait_runs_out_and_reports(scmx):
    L = scmx._lib
    flags = [torch.zeros(8, dtype=torch.int32, device="cuda") for _ in range(2)]
    peers = (ctypes.c_void_p * 8)(flags[0].data_ptr(), flags[1].data_ptr(), *([None] * 6))
    epoch = torch.zeros(1, dtype=torch.int32, device="cuda")
    status = L.status_buffer()
    status.zero_()
    L.call("scmx_set_wait_limit_ns", 2_000_000)
    try:
        t0 = time.perf_counter()
        L.call("scmx_peer_barrier", peers, 0, 2, L.ptr(epoch), L.ptr(status), L.stream())
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
    finally:
        L.call("scmx_set_wait_limit_ns", 2_000_000_000)
    assert dt < 1.0, f"the barrier took {dt:.3f} s with a 2 ms limit"
    assert status[0].item() == 20 and status[1].item() == 0      # code 20 = peer barrier, reported by rank 0
    assert epoch.item() == 1 and flags[1][0].item() == 1          # the rank still signalled its peer and moved on
    with pytest.raises(scmx._lib.ScmxError, match="peer barrier"):
        L.check_status()
    assert status[0].item() == 0                                  # check_status() clears the word
    # the context is still usable and a barrier of a world of one completes at once
    L.call("scmx_peer_barrier", peers, 0, 1, L.ptr(epoch), L.ptr(status), L.stream())
    torch.cuda.synchronize()
    L.check_status()
    assert epoch.item() == 2


def test_wait_limit_range(scmx):
    L = scmx._lib
    assert L.lib().scmx_set_wait_limit_ns(10) == -1
    assert L.lib().scmx_set_wait_limit_ns(2_000_000_000) == 0
