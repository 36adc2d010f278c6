"""GPU: the grouped GEMM entry point that brings its own scratch (scmx_moe_mm_static).

Some users of libscmx cannot allocate device memory when they call it: a serving process that gave the whole GPU to
its own memory pool at start-up, or a host runtime that binds the C ABI from another language and has no device
allocator.  scmx_moe_mm_static decodes expert weights into a fixed 16 MiB array inside the library instead of a
caller-provided buffer.  This test calls it through the C ABI twice in a row, with different inputs, and checks each
result bit for bit against scmx_moe_mm (the entry point that takes caller scratch); it also checks that a shape beyond
the built-in limit is refused.  Collected last so that a failure here cannot hide any other test.
"""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(scmx, seed, E, N, K, R):
    F = scmx.sc_format
    g = torch.Generator(device="cuda").manual_seed(seed)
    packs = [F.quantize_device((torch.randn((N, K), generator=g, device="cuda") * 0.02).contiguous(), want_qw=False)
             for _ in range(E)]
    codes = torch.stack([p[0] for p in packs])
    bcodes = torch.stack([p[1] for p in packs])
    ws = torch.stack([p[2] for p in packs])
    ex = torch.sort(torch.randint(0, E - 1, (R,), generator=g, device="cuda")).values.to(torch.int32)   # last expert empty
    off, ts, _ = scmx.sc_moe.segments(ex, E, 128)
    xq = torch.randint(-127, 128, (R + 128, K), dtype=torch.int8, device="cuda", generator=g)
    xs = torch.rand(R, generator=g, device="cuda") * 1e-2
    return codes, bcodes, ws, off, ts, xq, xs


def _static(scmx, xq, R, codes, bcodes, ws, off, ts, N, epi, xs, out):
    L = scmx._lib
    E, K = ws.shape[0], xq.shape[1]
    return L.lib().scmx_moe_mm_static(L.ptr(xq), R, L.ptr(codes), L.ptr(bcodes), L.ptr(ws), L.ptr(off), L.ptr(ts), E, N, K,
                                      scmx.sc_format.DEFAULT.c_struct(), epi, L.ptr(xs), L.ptr(out), 128,
                                      L.ptr(L.status_buffer()), L.stream())


def test_static_scratch_matches_caller_scratch_twice(scmx):
    M_ = scmx.sc_moe
    for seed, (E, N, K, R) in enumerate([(6, 512, 1024, 700), (5, 256, 2048, 333)]):
        codes, bcodes, ws, off, ts, xq, xs = _case(scmx, seed, E, N, K, R)
        for epi in (0, 1):
            ref = M_.moe_mm(xq, R, codes, bcodes, ws, off, ts, 0, N, epi, xs)
            out = torch.full_like(ref, -3)
            rc = _static(scmx, xq, R, codes, bcodes, ws, off, ts, N, epi, xs, out)
            assert rc == 0, scmx._lib.lib().scmx_last_error_string().decode()
            torch.cuda.synchronize()
            scmx._lib.check_status()
            assert torch.equal(out, ref), f"call {seed}, epi {epi}: static-scratch result differs"


def test_static_scratch_several_passes_and_swiglu(scmx):
    """N * K = 4 MiB and five experts: two experts fit one 8 MiB half, so the call runs three passes and uses both halves
    (the first one twice); then one call with the SwiGLU epilogue.  Bit for bit against scmx_moe_mm."""
    M_ = scmx.sc_moe
    E, N, K, R = 5, 2048, 2048, 900
    codes, bcodes, ws, off, ts, xq, xs = _case(scmx, 7, E, N, K, R)
    ex = torch.sort(torch.randint(0, E, (R,), device="cuda")).values.to(torch.int32)      # every expert, incl. the last pass's
    off, ts, _ = M_.segments(ex, E, 128)
    for epi in (1, 0, 3):
        ref = M_.moe_mm(xq, R, codes, bcodes, ws, off, ts, 0, N, epi, xs)
        out = torch.full_like(ref, -3)
        rc = _static(scmx, xq, R, codes, bcodes, ws, off, ts, N, epi, xs, out)
        assert rc == 0, scmx._lib.lib().scmx_last_error_string().decode()
        torch.cuda.synchronize()
        scmx._lib.check_status()
        assert torch.equal(out, ref), f"epi {epi}: static-scratch result differs over three passes"


def test_static_scratch_rejects_oversize(scmx):
    L = scmx._lib
    p = ctypes.c_void_p(256)
    rc = L.lib().scmx_moe_mm_static(p, 16, p, p, p, p, p, 2, 4096, 4096, scmx.sc_format.DEFAULT.c_struct(), 0, None, p, 128, p, None)
    assert rc == -5 and b"8388608" in L.lib().scmx_last_error_string()
