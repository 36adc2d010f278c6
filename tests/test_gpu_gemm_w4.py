"""GPU: the GEMMs that read packed 4-bit weights directly (scmx_mm_w4 / scmx_moe_mm_w4: tiles expanded to INT8 in shared memory
inside the K loop) against the oracle and against the two-kernel forms, bit for bit."""
import numpy as np
import pytest
import torch

from helpers import bf16_np, cuda, to_bf16_cuda

pytestmark = pytest.mark.gpu


def _pack(scmx, oracle, rng, N, K, fmt_kw):
    F = scmx.sc_format
    fmt = F.Format(**fmt_kw)
    ofmt = oracle.Format(fmt.block, fmt.code_mag, fmt.mult, fmt.bc_bits)
    c4 = rng.integers(0, 16, (N, K)).astype(np.uint8)
    bcode = rng.integers(0, len(fmt.mult), (N, K // fmt.block)).astype(np.uint8)
    ws = (np.abs(rng.standard_normal(N)) * 1e-3 + 1e-5).astype(np.float32)
    codes, bc, ws = F.pack_rows(c4, bcode, ws, fmt)
    return fmt, codes, bc, ws, oracle.decode(codes, bc, N, K, ofmt)


@pytest.mark.parametrize("fmt_kw", [dict(), dict(block=16), dict(block=16, mult=(1, 2, 3, 4, 5, 6, 8, 10), bc_bits=4),
                                    dict(block=32, mult=(1, 2, 3, 4)), dict(block=8),
                                    dict(block=32, code_mag=(0, 1, 2, 3, 4, 5, 6, 7), mult=(1, 3, 9, 15))])
@pytest.mark.parametrize("M,N,K", [(128, 256, 128), (256, 384, 2048), (384, 1024, 1024), (512, 2048, 6144), (640, 96, 256)])
def test_dense_from_packed_exact(scmx, oracle, M, N, K, fmt_kw):
    S, F = scmx.sc_kernels, scmx.sc_format
    rng = np.random.default_rng(M + N + K)
    fmt, codes, bc, ws, q = _pack(scmx, oracle, rng, N, K, fmt_kw)
    xq = rng.integers(-127, 128, (M, K)).astype(np.int8)
    xs = (np.abs(rng.standard_normal(M)) * 1e-3).astype(np.float32)
    res = oracle.bf16_round(rng.standard_normal((M, N)).astype(np.float32))
    acc = oracle.gemm_i32(xq, q)
    S.set_format(fmt)
    try:
        c, b, s = F.to_device(codes, bc, ws)
        dx, dxs = cuda(xq), cuda(xs)
        assert np.array_equal(S.mm_w4_epi(dx, c, b, None, None, N, 0).cpu().numpy(), acc)
        assert np.array_equal(bf16_np(S.mm_w4_epi(dx, c, b, dxs, s, N, 1)), oracle.epilogue(acc, xs, ws, 1))
        assert np.array_equal(bf16_np(S.mm_w4_epi(dx, c, b, dxs, s, N, 2, res=to_bf16_cuda(res))), oracle.epilogue(acc, xs, ws, 2, res))
        if N % 64 == 0:
            wq = S.unpack_i8(c, b, N, K)
            assert torch.equal(S.mm_w4_epi(dx, c, b, dxs, s, N, 3), S.mm_epi(dx, wq, dxs, s, 3))
        torch.cuda.synchronize()
        scmx._lib.check_status()
    finally:
        S.set_format(F.Format())


@pytest.mark.parametrize("R", [1500, 3300])
@pytest.mark.parametrize("fmt_kw", [dict(), dict(block=16)])
def test_grouped_from_packed_exact(scmx, oracle, fmt_kw, R):
    """Eight experts, two of them empty, segment ends inside tiles (e2e/sc_moe.py:209-244), all epilogues, against the oracle
    and against the scratch-based form.  R = 1500: tiles of 256 rows; R = 3300 (more than 256 rows per expert on average):
    super tiles of 512 rows whose second row tile is skipped where a segment ends inside the first."""
    S, M_, F = scmx.sc_kernels, scmx.sc_moe, scmx.sc_format
    rng = np.random.default_rng(3)
    E, N, K = 8, 512, 1024
    packs = [_pack(scmx, oracle, rng, N, K, fmt_kw) for _ in range(E)]
    fmt = packs[0][0]
    ex = rng.integers(0, E, R)
    ex[ex == 3] = 2
    ex[ex == 7] = 0
    ex = np.sort(ex).astype(np.int32)
    xq = rng.integers(-127, 128, (R, K)).astype(np.int8)
    xs = (np.abs(rng.standard_normal(R)) * 1e-3).astype(np.float32)
    S.set_format(fmt)
    try:
        codes = torch.stack([F.to_device(p[1], p[2], p[3])[0] for p in packs])
        bcs = torch.stack([F.to_device(p[1], p[2], p[3])[1] for p in packs])
        wss = torch.stack([F.to_device(p[1], p[2], p[3])[2] for p in packs])
        off, ts, mt = M_.segments(cuda(ex), E, 128)
        xp = cuda(np.concatenate([xq, np.zeros((128, K), np.int8)]))
        dxs = cuda(xs)
        off_n = off.cpu().numpy()
        qs, wsl = [p[4] for p in packs], [p[3] for p in packs]
        for epi in (0, 1, 3):
            got = M_.moe_mm(xp, R, codes, bcs, wss, off, ts, mt, N, epi, dxs)
            want = oracle.moe_mm(xq, R, qs, off_n, epi, xs, wsl)
            got_n = got.cpu().numpy() if epi == 0 else bf16_np(got)
            if epi == 3:
                bad = np.flatnonzero((got_n != want).ravel())
                assert bad.size <= 4
            else:
                assert np.array_equal(got_n, want), epi
            M_.FUSED_UNPACK = False
            try:
                assert torch.equal(got, M_.moe_mm(xp, R, codes, bcs, wss, off, ts, mt, N, epi, dxs))
            finally:
                M_.FUSED_UNPACK = True
        torch.cuda.synchronize()
        scmx._lib.check_status()
    finally:
        S.set_format(F.Format())
