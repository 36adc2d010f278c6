"""GPU: the streaming (bulk-copy ring, persistent CTAs) form of the decode GEMV, forced on small and ragged shapes and run
on one matrix above its automatic threshold, against the oracle's exact integer totals and epilogues, as the reference
checks every shape it times (e2e/sc_decode.py:241-270).  Also the list form (scmx_gemv_multi): many independent GEMVs in
one launch."""
import numpy as np
import pytest
import torch

from helpers import bf16_np, cuda, to_bf16_cuda

pytestmark = pytest.mark.gpu


@pytest.fixture
def stream_always(scmx):
    scmx._lib.call("scmx_set_gemv_stream", 2)
    yield
    scmx._lib.call("scmx_set_gemv_stream", 1)


def _random_pack(scmx, oracle, rng, N, K, fmt_kw):
    F = scmx.sc_format
    fmt = F.Format(**fmt_kw)
    ofmt = oracle.Format(fmt.block, fmt.code_mag, fmt.mult, fmt.bc_bits)
    c4 = rng.integers(0, 16, (N, K)).astype(np.uint8)
    bcode = rng.integers(0, len(fmt.mult), (N, K // fmt.block)).astype(np.uint8)
    ws = (np.abs(rng.standard_normal(N)) * 1e-3 + 1e-5).astype(np.float32)
    codes, bc, ws = F.pack_rows(c4, bcode, ws, fmt)
    return fmt, codes, bc, ws, oracle.decode(codes, bc, N, K, ofmt)


SHAPES = [(64, 1024), (100, 2048), (2048, 2048), (516, 6144), (40, 8192), (4, 2048), (1028, 1024)]


@pytest.mark.parametrize("fmt_kw", [dict(), dict(block=16), dict(block=32, mult=(1, 2, 3, 4)), dict(block=8),
                                    dict(block=16, mult=(1, 2, 3, 4, 5, 6, 8, 10), bc_bits=4), dict(block=64)])
@pytest.mark.parametrize("N,K", SHAPES)
def test_streaming_gemv_small_and_ragged(scmx, oracle, stream_always, N, K, fmt_kw):
    G, S, F = scmx.sc_decode, scmx.sc_kernels, scmx.sc_format
    rng = np.random.default_rng(N * 7 + K)
    fmt, codes, bc, ws, q = _random_pack(scmx, oracle, rng, N, K, fmt_kw)
    xq = rng.integers(-127, 128, K).astype(np.int8)
    xq[:16] = 127
    xs = np.array([0.0123], np.float32)
    res = oracle.bf16_round(rng.standard_normal(N).astype(np.float32))
    S.set_format(fmt)
    try:
        c, b, s = F.to_device(codes, bc, ws)
        dx, dxs = cuda(xq), cuda(xs)
        tot = G.gemv(dx, c, b, dxs, s, N, 0)
        assert np.array_equal(tot.cpu().numpy(), oracle.gemv_i32(xq, q))
        y1 = G.gemv(dx, c, b, dxs, s, N, 1)
        assert np.array_equal(bf16_np(y1), oracle.gemv(xq, xs[0], q, ws, 1))
        y2 = G.gemv(dx, c, b, dxs, s, N, 2, res=to_bf16_cuda(res))
        assert np.array_equal(bf16_np(y2), oracle.gemv(xq, xs[0], q, ws, 2, res))
        y3 = G.gemv(dx, c, b, dxs, s, N, 3)           # rows read as interleaved [g, g, u, u] groups
        o1 = oracle.gemv(xq, xs[0], q, ws, 1).reshape(N // 4, 4)
        want = oracle.swiglu_bf16(o1[:, :2].reshape(-1), o1[:, 2:].reshape(-1))
        assert np.array_equal(bf16_np(y3), want)
        torch.cuda.synchronize()
        scmx._lib.check_status()
    finally:
        S.set_format(F.Format())


def test_streaming_gemv_above_threshold(scmx, oracle):
    """16384 x 2048 = 16 MiB of packed codes: the automatic choice (no switch set) is the streaming kernel."""
    G, F = scmx.sc_decode, scmx.sc_format
    rng = np.random.default_rng(11)
    N, K = 16384, 2048
    _, codes, bc, ws, q = _random_pack(scmx, oracle, rng, N, K, dict())
    xq = rng.integers(-127, 128, K).astype(np.int8)
    xs = np.array([0.02], np.float32)
    c, b, s = F.to_device(codes, bc, ws)
    tot = G.gemv(cuda(xq), c, b, cuda(xs), s, N, 0)
    assert np.array_equal(tot.cpu().numpy(), oracle.gemv_i32(xq, q))
    y = G.gemv(cuda(xq), c, b, cuda(xs), s, N, 1)
    assert np.array_equal(bf16_np(y), oracle.gemv(xq, xs[0], q, ws, 1))
    scmx._lib.call("scmx_set_gemv_stream", 0)          # the register kernel gives the same bits
    try:
        assert torch.equal(G.gemv(cuda(xq), c, b, cuda(xs), s, N, 1), y)
    finally:
        scmx._lib.call("scmx_set_gemv_stream", 1)
    scmx._lib.check_status()


def test_gemv_stream_switch_rejects_other_values(scmx):
    L = scmx._lib
    assert L.lib().scmx_set_gemv_stream(3) == -1
    assert L.lib().scmx_set_gemv_stream(-1) == -1
    assert L.lib().scmx_set_gemv_stream(1) == 0


def test_gemv_list_one_launch(scmx, oracle):
    """Nine independent GEMVs of mixed shapes and epilogues in one launch, each against the oracle, twice (the ring and the
    split-K sums must be clean for the second launch)."""
    G, F = scmx.sc_decode, scmx.sc_format
    rng = np.random.default_rng(21)
    shapes = [(256, 2048, 1), (132, 6144, 2), (512, 1024, 3), (64, 8192, 0), (2048, 2048, 3), (4, 1024, 1), (772, 2048, 2),
              (100, 4096, 1), (1024, 3072, 0)]
    jobs, want = [], []
    for N, K, epi in shapes:
        _, codes, bc, ws, q = _random_pack(scmx, oracle, rng, N, K, dict())
        xq = rng.integers(-127, 128, K).astype(np.int8)
        xq[:16] = 127
        xs = np.array([rng.uniform(0.005, 0.02)], np.float32)
        res = oracle.bf16_round(rng.standard_normal(N).astype(np.float32))
        c, b, s = F.to_device(codes, bc, ws)
        jobs.append((cuda(xq), c, b, cuda(xs), s, N, epi, to_bf16_cuda(res) if epi == 2 else None))
        if epi == 0:
            want.append(oracle.gemv_i32(xq, q))
        elif epi == 3:
            o1 = oracle.gemv(xq, xs[0], q, ws, 1).reshape(N // 4, 4)
            want.append(oracle.swiglu_bf16(o1[:, :2].reshape(-1), o1[:, 2:].reshape(-1)))
        else:
            want.append(oracle.gemv(xq, xs[0], q, ws, epi, res if epi == 2 else None))
    gl = G.GemvList(jobs)
    for _ in range(2):
        for o in gl.outs:
            o.fill_(-7)
        outs = gl.run()
        torch.cuda.synchronize()
        scmx._lib.check_status()
        for (N, K, epi), o, w in zip(shapes, outs, want):
            got = o.cpu().numpy() if epi == 0 else bf16_np(o)
            assert np.array_equal(got, w), (N, K, epi)


def test_gemv_list_refuses_unplanned_and_bad_jobs(scmx):
    L = scmx._lib
    jobs = (L.ScmxGemvJob * 2)()
    fmt = scmx.sc_format.DEFAULT.c_struct()
    st = L.status_buffer()
    import ctypes
    assert L.lib().scmx_gemv_multi(ctypes.byref(jobs), L.ptr(st), 2, fmt, L.ptr(st), 0, None) == -1     # not planned
    assert L.lib().scmx_gemv_multi_plan(ctypes.byref(jobs), 2, fmt) == -1                               # NULL pointers
    assert L.lib().scmx_gemv_multi_plan(ctypes.byref(jobs), 0, fmt) == -1
