"""GPU parity: the tcgen05 INT8 GEMM (dense and grouped) and the decode GEMV against the oracle.
INT32 accumulators are compared bit for bit; bf16 epilogue outputs bit for bit against the oracle's restatement
(and additionally within 1e-3 relative L2, the tolerance stated for floating-point outputs)."""
import numpy as np
import pytest
import torch

from helpers import bf16_np, cuda, llm_acts, llm_weights, rel_l2, sha, to_bf16_cuda

pytestmark = pytest.mark.gpu


def _status_ok(scmx):
    scmx._lib.check_status()


@pytest.mark.parametrize("bn", [0, 128, 256])
@pytest.mark.parametrize("M,N,K", [(256, 384, 2048), (128, 32, 16), (128, 256, 128), (384, 1024, 2064), (512, 2048, 6144)])
def test_mm_i8_i32_exact(scmx, oracle, bn, M, N, K):
    rng = np.random.default_rng(M + N + K)
    xq = rng.integers(-127, 128, (M, K)).astype(np.int8)
    wq = rng.integers(-96, 97, (N, K)).astype(np.int8)
    scmx.sc_kernels.set_gemm_tile(bn)
    try:
        acc = scmx.sc_kernels.mm_i8_i32(cuda(xq), cuda(wq))
        _status_ok(scmx)
    finally:
        scmx.sc_kernels.set_gemm_tile(0)
    assert np.array_equal(acc.cpu().numpy(), oracle.gemm_i32(xq, wq))


def test_mm_i8_ragged_rows_through_abi(scmx, oracle):
    """M = 200 (not a tile multiple) straight through the C ABI: rows beyond M are neither read nor written."""
    rng = np.random.default_rng(0)
    M, N, K = 200, 1024, 2048
    xq = rng.integers(-127, 128, (M, K)).astype(np.int8)
    wq = rng.integers(-96, 97, (N, K)).astype(np.int8)
    L = scmx._lib
    out = torch.full((256, N), -7, dtype=torch.int32, device="cuda")
    L.call("scmx_mm_i8", L.ptr(cuda(xq)), L.ptr(cuda(wq)), M, N, K, 0, None, None, None, L.ptr(out),
           L.ptr(L.status_buffer()), L.stream())
    _status_ok(scmx)
    assert np.array_equal(out[:M].cpu().numpy(), oracle.gemm_i32(xq, wq)) and bool((out[M:] == -7).all())


def test_extreme_accumulators(scmx, oracle):
    """All operands at their extremes: |acc| = 127 * 96 * K, the largest the format can produce."""
    M, N, K = 128, 64, 6144
    xq = np.full((M, K), 127, np.int8)
    xq[1::2] = -127
    wq = np.full((N, K), 96, np.int8)
    wq[::3] = -96
    acc = scmx.sc_kernels.mm_i8_i32(cuda(xq), cuda(wq))
    _status_ok(scmx)
    assert np.array_equal(acc.cpu().numpy(), oracle.gemm_i32(xq, wq))
    assert int(np.abs(acc.cpu().numpy()).max()) == 127 * 96 * K


@pytest.mark.parametrize("M,N,K", [(256, 512, 1024), (128, 256, 2048), (384, 768, 512)])
def test_mm_epi_against_oracle(scmx, oracle, M, N, K):
    """EPI 1 / 2 / 3 (e2e/test_sc_kernels.py:121-142)."""
    S = scmx.sc_kernels
    rng = np.random.default_rng(1)
    xq = rng.integers(-127, 128, (M, K)).astype(np.int8)
    wq = rng.integers(-96, 97, (N, K)).astype(np.int8)
    xs = (np.abs(rng.standard_normal(M)) * 1e-3).astype(np.float32)
    ws = (np.abs(rng.standard_normal(N)) * 1e-4).astype(np.float32)
    res = oracle.bf16_round(rng.standard_normal((M, N)).astype(np.float32))
    acc = oracle.gemm_i32(xq, wq)
    dx, dw, dxs, dws = cuda(xq), cuda(wq), cuda(xs), cuda(ws)
    y1 = bf16_np(S.mm_epi(dx, dw, dxs, dws, 1))
    y2 = bf16_np(S.mm_epi(dx, dw, dxs, dws, 2, res=to_bf16_cuda(res)))
    perm = S.interleave_gate_up(N // 2)
    y3 = bf16_np(S.mm_epi(dx, cuda(wq[perm]), dxs, cuda(ws[perm]), 3))
    _status_ok(scmx)
    o1 = oracle.epilogue(acc, xs, ws, 1)
    assert np.array_equal(y1, o1) and rel_l2(y1, o1) <= 1e-3
    assert np.array_equal(y2, oracle.epilogue(acc, xs, ws, 2, res))
    o3 = oracle.swiglu_bf16(o1[:, :N // 2], o1[:, N // 2:])      # gate = first half, up = second half of the unpermuted GEMM
    assert y3.shape == (M, N // 2)
    bad = np.flatnonzero((y3 != o3).ravel())
    gates = np.abs(o1[:, :N // 2].ravel()[bad])
    assert set(gates.tolist()) <= {6.84375} and rel_l2(y3, o3) <= 1e-3


def test_headline_single_layer(scmx, oracle, digests):
    """Config 1: W [6144, 2048] ~ N(0, 0.02), X [512, 2048] bf16 with 8 outlier channels: packed codes, activation
    codes and INT32 accumulators equal the digests recorded from the reference's NumPy path; Y within 1e-3 rel-L2."""
    import ml_dtypes  # noqa: F401  (only to mirror the generator's bf16 rounding)
    S, F = scmx.sc_kernels, scmx.sc_format
    r0 = np.random.default_rng(0)
    W = (r0.standard_normal((6144, 2048)) * 0.02).astype(np.float32)
    X = r0.standard_normal((512, 2048))
    cols = r0.choice(2048, 8, replace=False)
    X[:, cols] *= 20
    X = oracle.bf16_round(X.astype(np.float32))
    if sha(W) != digests["W"] or sha(X) != digests["X"]:
        pytest.skip("NumPy's generator stream differs from the one the digests were recorded with")
    codes, bc, ws, qw, _ = F.quantize_device(cuda(W))
    xq, xs = S.act_quant(to_bf16_cuda(X))
    wq = S.unpack_i8(codes, bc, 6144, 2048)
    acc = S.mm_i8_i32(xq, wq)
    y = S.mm_epi(xq, wq, xs, ws, 1)
    _status_ok(scmx)
    assert sha(codes.cpu().numpy()) == digests["codes"] and sha(bc.cpu().numpy()) == digests["bcodes"]
    assert sha(ws.cpu().numpy()) == digests["wscale"]
    assert sha(xq.cpu().numpy()) == digests["xq"] and sha(xs.cpu().numpy()) == digests["xs"]
    assert sha(acc.cpu().numpy()) == digests["acc"]
    yref = acc.cpu().numpy().astype(np.float64) * xs.cpu().numpy().astype(np.float64)[:, None] * ws.cpu().numpy().astype(np.float64)[None]
    assert rel_l2(bf16_np(y), yref) <= 4e-3      # bf16 rounding of the output itself is 2^-9 relative
    assert np.array_equal(bf16_np(y), oracle.epilogue(acc.cpu().numpy(), xs.cpu().numpy(), ws.cpu().numpy(), 1))


def test_w4a8_linear_module(scmx, oracle):
    """W4A8Linear on M = 200 rows (padding path), e2e/w4a8_mlx.py:218-239."""
    rng = np.random.default_rng(0)
    M, N, K = 200, 1024, 2048
    w = llm_weights(rng, N, K)
    x = llm_acts(rng, M, K, oracle)
    codes, shifts, wscale = scmx.w4a8.pack_linear(w)
    for resident in (False, True):
        lin = scmx.w4a8.W4A8Linear(codes, shifts, wscale, resident_int8=resident)
        y = bf16_np(lin(to_bf16_cuda(x)))
        _status_ok(scmx)
        r = oracle.quantize_rows(w)
        assert np.array_equal(lin.int8_weight().cpu().numpy(), r["qw"])
        xq, xs = oracle.act_quant(x)
        assert np.array_equal(y, oracle.epilogue(oracle.gemm_i32(xq, r["qw"]), xs, r["wscale"], 1))


def test_full_size_checksum(scmx):
    """Qwen3-1.7B-shaped gate|up GEMM at full size (2048 x 12288 x 2048): row and column checksums of the INT32
    accumulators equal the ones computed from the operands' sums (exact integer identities), and the library GEMM
    torch._int_mm agrees element for element."""
    g = torch.Generator(device="cuda").manual_seed(0)
    M, N, K = 2048, 12288, 2048
    xq = torch.randint(-127, 128, (M, K), dtype=torch.int8, device="cuda", generator=g)
    wq = torch.randint(-96, 97, (N, K), dtype=torch.int8, device="cuda", generator=g)
    acc = scmx.sc_kernels.mm_i8_i32(xq, wq)
    _status_ok(scmx)
    colsum = wq.to(torch.int64).sum(0)
    assert torch.equal(acc.to(torch.int64).sum(1), (xq.to(torch.int64) * colsum).sum(1))
    rowsum = xq.to(torch.int64).sum(0)
    assert torch.equal(acc.to(torch.int64).sum(0), (wq.to(torch.int64) * rowsum).sum(1))
    assert torch.equal(acc, torch._int_mm(xq, wq.t()))


# ---------------------------------------------------------------------------------------------------------------------
def _moe_case(oracle, scmx, E, N, K, R, seed=0):
    rng = np.random.default_rng(seed)
    p = np.r_[0.4, np.full(E - 2, 0.6 / (E - 2))] if E > 2 else np.array([1.0])
    ex = np.sort(rng.choice(E - 1 if E > 2 else 1, R, p=p))       # last expert empty
    if E > 4:
        ex[ex == 3] = 2                                             # expert 3 empty
    packs = [oracle.quantize(rng.standard_normal((N, K)) * 0.02) for _ in range(E)]
    xq = rng.integers(-127, 128, (R, K)).astype(np.int8)
    xs = (np.abs(rng.standard_normal(R)) * 1e-2).astype(np.float32)
    off = np.concatenate([[0], np.cumsum(np.bincount(ex, minlength=E))]).astype(np.int32)
    return ex, packs, xq, xs, off


@pytest.mark.parametrize("E,N,K,R", [(8, 256, 512, 600), (4, 512, 1024, 1000), (8, 128, 256, 50)])
def test_grouped_gemm_uneven_segments(scmx, oracle, E, N, K, R):
    """Grouped GEMM vs per-expert integer GEMMs, uneven segments including empty experts (e2e/sc_moe.py:209-244):
    from packed weights and from pre-unpacked INT8, EPI 0 / 1 / 3."""
    M_, F = scmx.sc_moe, scmx.sc_format
    ex, packs, xq, xs, off = _moe_case(oracle, scmx, E, N, K, R)
    codes = torch.stack([F.to_device(*p[:3])[0] for p in packs])
    bcodes = torch.stack([F.to_device(*p[:3])[1] for p in packs])
    ws = torch.stack([F.to_device(*p[:3])[2] for p in packs])
    qw = [p[3] for p in packs]
    wsn = [p[2] for p in packs]
    doff, dts, mt = M_.segments(cuda(ex.astype(np.int32)), E, 128)
    assert np.array_equal(doff.cpu().numpy(), off)
    xqp = cuda(np.concatenate([xq, np.zeros((128, K), np.int8)]))
    ref0 = oracle.moe_mm(xq, R, qw, off, 0)
    ref1 = oracle.moe_mm(xq, R, qw, off, 1, xs, wsn)
    perm = scmx.sc_kernels.interleave_gate_up(N // 2)
    ref3 = oracle.moe_mm(xq, R, [q[perm] for q in qw], off, 3, xs, [w[perm] for w in wsn])
    wq8 = M_.unpack_experts(codes, bcodes, N, K)
    for old in (1, 3, 8):
        M_.EXPERTS_PER_PASS = old
        a0 = M_.moe_mm(xqp, R, codes, bcodes, ws, doff, dts, mt, N, 0)
        assert np.array_equal(a0.cpu().numpy(), ref0), f"experts_per_pass={old}"
    M_.EXPERTS_PER_PASS = 8
    a0b = M_.moe_mm_i8(xqp, R, wq8, ws, doff, dts, mt, N, 0)
    y1 = M_.moe_mm(xqp, R, codes, bcodes, ws, doff, dts, mt, N, 1, cuda(xs))
    y1b = M_.moe_mm_i8(xqp, R, wq8, ws, doff, dts, mt, N, 1, cuda(xs))
    cp = torch.stack([c.reshape(N, -1)[cuda(perm)].reshape(-1) for c in codes])
    y3 = M_.moe_mm(xqp, R, cp, bcodes[:, cuda(perm)], ws[:, cuda(perm)], doff, dts, mt, N, 3, cuda(xs))
    _status_ok(scmx)
    assert np.array_equal(a0b.cpu().numpy(), ref0)
    assert np.array_equal(bf16_np(y1), ref1) and np.array_equal(bf16_np(y1b), ref1)
    bad = (bf16_np(y3) != ref3).sum()
    assert bad <= 2 and rel_l2(bf16_np(y3), ref3) <= 1e-3


def test_grouped_gemm_single_expert_equals_dense(scmx, oracle):
    rng = np.random.default_rng(3)
    N, K, R = 256, 512, 384
    xq = rng.integers(-127, 128, (R, K)).astype(np.int8)
    wq = rng.integers(-96, 97, (N, K)).astype(np.int8)
    off = cuda(np.array([0, R], np.int32))
    ts = cuda(np.array([0, 3], np.int32))
    xqp = cuda(np.concatenate([xq, np.zeros((128, K), np.int8)]))
    a = scmx.sc_moe.moe_mm_i8(xqp, R, cuda(wq), torch.ones((1, N), device="cuda"), off, ts, 4, N, 0)
    _status_ok(scmx)
    assert np.array_equal(a.cpu().numpy(), oracle.gemm_i32(xq, wq))


def test_moe_block_end_to_end(scmx, oracle):
    """One MoE half-block the way e2e/fused_olmoe.py:211-245 chains it: router -> route_sort -> gather -> gate|up grouped
    GEMM with SwiGLU -> act_quant -> down grouped GEMM -> combine, against the oracle's chain."""
    S, M_, F = scmx.sc_kernels, scmx.sc_moe, scmx.sc_format
    rng = np.random.default_rng(8)
    L, D, Fd, E, k = 300, 512, 256, 8, 2
    Mp = S.pad_rows(L)
    h = oracle.bf16_round(rng.standard_normal((Mp, D)).astype(np.float32))
    h[L:] = 0
    nw = oracle.bf16_round(rng.lognormal(0, 0.3, D).astype(np.float32))
    logits = rng.standard_normal((L, E)).astype(np.float32)
    perm = S.interleave_gate_up(Fd)
    gu = [oracle.quantize(rng.standard_normal((2 * Fd, D)) * 0.02) for _ in range(E)]
    dn = [oracle.quantize(rng.standard_normal((D, Fd)) * 0.02) for _ in range(E)]

    def stack(packs, p=None):
        c = np.stack([x[0].reshape(x[1].shape[0], -1)[p if p is not None else slice(None)].reshape(-1) for x in packs])
        b = np.stack([x[1][p if p is not None else slice(None)] for x in packs])
        s = np.stack([x[2][p if p is not None else slice(None)] for x in packs])
        return F.to_device(c, b, s)
    cg, bg, sg = stack(gu, perm)
    cd, bd, sd = stack(dn)
    # ---- device chain
    xq, xs, xn = S.rmsnorm_quant_n(to_bf16_cuda(h), to_bf16_cuda(nw), 1e-5)
    inds, scores = M_.router_topk(cuda(logits), k)
    pos, tok, es, off, ts, mt = M_.route_sort(inds, E, 128)
    R = L * k
    xq_s, xs_s = M_.gather_rows(xq, xs, tok, R)
    act = M_.moe_mm(xq_s, R, cg, bg, sg, off, ts, mt, 2 * Fd, 3, xs_s)
    xq2, xs2 = S.act_quant(act, R + 128)
    yd = M_.moe_mm(xq2, R, cd, bd, sd, off, ts, mt, D, 1, xs2)
    hout, xqn, xsn = M_.moe_combine(yd, pos, scores, to_bf16_cuda(h), to_bf16_cuda(nw), 1e-5, L)
    _status_ok(scmx)
    # ---- oracle chain, driven by the device's routing decisions (order inside a segment is arbitrary)
    oxq, oxs, _ = oracle.rmsnorm_quant(h[:L], nw, 1e-5, Mp)
    assert np.array_equal(xq.cpu().numpy(), oxq)
    pos_n, tok_n, off_n = pos.cpu().numpy(), tok.cpu().numpy(), off.cpu().numpy()
    assert oracle.check_route(inds.cpu().numpy(), E, 128, pos_n, tok_n, es.cpu().numpy(), off_n, ts.cpu().numpy())
    a = oracle.moe_mm(oxq[tok_n[:R]], R, [g[3][perm] for g in gu], off_n, 3, oxs[tok_n[:R]], [g[2][perm] for g in gu])
    assert rel_l2(bf16_np(act), a) <= 1e-3
    a_dev = bf16_np(act)                      # continue from the device's activations so later stages compare bit for bit
    oq2, os2 = oracle.act_quant(a_dev)
    assert np.array_equal(xq2[:R].cpu().numpy(), oq2) and not xq2[R:].any()
    oyd = oracle.moe_mm(oq2, R, [d[3] for d in dn], off_n, 1, os2, [d[2] for d in dn])
    assert np.array_equal(bf16_np(yd), oyd)
    oh = oracle.moe_combine(oyd, pos_n, bf16_np(scores), h, L)
    assert np.array_equal(bf16_np(hout), oh)


# ---------------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("N,K", [(256, 2048), (512, 6144), (64, 1024), (2048, 2048), (128, 128), (12288, 2048)])
def test_gemv_against_oracle(scmx, oracle, N, K):
    """GEMV == exact integer totals + the GEMM's epilogues; xq[:16] = 127 stresses the largest partial sums
    (e2e/sc_decode.py:241-270)."""
    G, S, F = scmx.sc_decode, scmx.sc_kernels, scmx.sc_format
    rng = np.random.default_rng(N + K)
    rows = min(N, 512)
    w = llm_weights(rng, rows, K, 0.5)
    oc, ob, ows, oqw = oracle.quantize(w)
    reps = N // rows
    oc2 = np.tile(oc.reshape(rows, -1), (reps, 1)).reshape(-1)
    ob2, ows2, oqw2 = np.tile(ob, (reps, 1)), np.tile(ows, reps), np.tile(oqw, (reps, 1))
    c, b, s = F.to_device(oc2, ob2, ows2)
    xq = rng.integers(-127, 128, K).astype(np.int8)
    xq[:16] = 127
    xs = np.array([0.01], np.float32)
    tot = G.gemv(cuda(xq), c, b, cuda(xs), s, N, 0)
    assert np.array_equal(tot.cpu().numpy(), oracle.gemv_i32(xq, oqw2))
    y1 = G.gemv(cuda(xq), c, b, cuda(xs), s, N, 1)
    assert np.array_equal(bf16_np(y1), oracle.gemv(xq, xs[0], oqw2, ows2, 1))
    res = oracle.bf16_round(rng.standard_normal(N).astype(np.float32))
    y2 = G.gemv(cuda(xq), c, b, cuda(xs), s, N, 2, res=to_bf16_cuda(res))
    assert np.array_equal(bf16_np(y2), oracle.gemv(xq, xs[0], oqw2, ows2, 2, res))
    perm = S.interleave_gate_up(N // 2)
    cp, bp, sp = F.to_device(oc2.reshape(N, -1)[perm].reshape(-1), ob2[perm], ows2[perm])
    y3 = G.gemv(cuda(xq), cp, bp, cuda(xs), sp, N, 3)
    o1 = oracle.gemv(xq, xs[0], oqw2, ows2, 1)
    assert np.array_equal(bf16_np(y3), oracle.swiglu_bf16(o1[:N // 2], o1[N // 2:]))
    # GEMV and GEMM compute the same bits
    acc = S.mm_i8_i32(cuda(np.tile(xq, (128, 1))), cuda(oqw2))
    assert torch.equal(acc[0], tot)


def test_gemv_prologues_and_gather(scmx, oracle):
    G, S, F = scmx.sc_decode, scmx.sc_kernels, scmx.sc_format
    rng = np.random.default_rng(5)
    N, K = 512, 2048
    c, b, s, qw = (None,) * 4
    oc, ob, ows, oqw = oracle.quantize(rng.standard_normal((N, K)) * 0.02)
    c, b, s = F.to_device(oc, ob, ows)
    x = oracle.bf16_round((rng.standard_normal((1, K)) * rng.lognormal(0, 1, K)).astype(np.float32))
    nw = oracle.bf16_round(rng.lognormal(0, 0.3, K).astype(np.float32))
    dx, dnw = to_bf16_cuda(x), to_bf16_cuda(nw)
    for pro, (q_, s_) in ((1, S.act_quant(dx, 1)), (2, S.rmsnorm_quant(dx, dnw, 1e-6, 1))):
        y0 = G.gemv(q_, c, b, s_, s, N, 1)
        y1 = G.gemv(dx, c, b, None, s, N, 1, pro=pro, nw=dnw, eps=1e-6)
        assert torch.equal(y0, y1)
    # MoE gather: 3 experts, slots (2, 0) with per-slot inputs, then a shared expert slot
    E, N, K = 3, 256, 1024
    packs = [oracle.quantize(rng.standard_normal((N, K)) * 0.02) for _ in range(E)]
    cE = torch.stack([F.to_device(*p[:3])[0] for p in packs])
    bE = torch.stack([F.to_device(*p[:3])[1] for p in packs])
    sE = torch.stack([F.to_device(*p[:3])[2] for p in packs])
    xq = rng.integers(-127, 128, (3, K)).astype(np.int8)
    xs = np.array([0.01, 0.02, 0.03], np.float32)
    y = G.gemv(cuda(xq), cE, bE, cuda(xs), sE, N, 1, eidx=cuda(np.array([2, 0], np.int32)), xstride=1)
    for j, e in enumerate((2, 0)):
        assert np.array_equal(bf16_np(y[j]), oracle.gemv(xq[j], xs[j], packs[e][3], packs[e][2], 1))
    y = G.gemv(cuda(xq), cE, bE, cuda(xs), sE, N, 1, eidx=cuda(np.array([2, 0], np.int32)), xstride=1, shared=1)
    assert y.shape == (3, N)
    assert np.array_equal(bf16_np(y[2]), oracle.gemv(xq[2], xs[2], packs[1][3], packs[1][2], 1))
    y = G.gemv(cuda(xq[0]), cE, bE, cuda(xs[:1]), sE, N, 1, eidx=cuda(np.array([1, 2], np.int32)), xstride=0)
    assert np.array_equal(bf16_np(y[1]), oracle.gemv(xq[0], xs[0], packs[2][3], packs[2][2], 1))


FORMATS = [dict(), dict(block=16), dict(block=32, mult=(1, 2, 3, 4)),
           dict(block=16, mult=(1, 2, 3, 4, 5, 6, 8, 10), bc_bits=4),
           dict(block=32, code_mag=(0, 1, 2, 3, 4, 5, 6, 7), mult=(1, 3, 9, 15))]


@pytest.mark.parametrize("kw", FORMATS)
def test_other_formats_gemv_and_grouped_gemm(scmx, oracle, kw):
    """The reference's e2e/test_formats.py: random codes of five formats through the GEMV and the grouped GEMM."""
    S, G, M_, F = scmx.sc_kernels, scmx.sc_decode, scmx.sc_moe, scmx.sc_format
    fmt = F.Format(**kw)
    ofmt = oracle.Format(fmt.block, fmt.code_mag, fmt.mult, fmt.bc_bits)
    rng = np.random.default_rng(0)
    N, K, M = 256, 2048, 128
    c4 = rng.integers(0, 16, (N, K)).astype(np.uint8)
    bcode = rng.integers(0, len(fmt.mult), (N, K // fmt.block)).astype(np.uint8)
    ws = (np.abs(rng.standard_normal(N)) * 1e-3).astype(np.float32)
    codes, bc, ws = F.pack_rows(c4, bcode, ws, fmt)
    q = oracle.decode(codes, bc, N, K, ofmt)
    xq = rng.integers(-127, 128, (M, K)).astype(np.int8)
    S.set_format(fmt)
    try:
        c, b, s = F.to_device(codes, bc, ws)
        tot = G.gemv(cuda(xq[0]), c, b, cuda(np.array([1e-2], np.float32)), s, N, 0)
        assert np.array_equal(tot.cpu().numpy(), oracle.gemv_i32(xq[0], q))
        y = G.gemv(cuda(xq[0]), c, b, cuda(np.array([1e-2], np.float32)), s, N, 1)
        assert np.array_equal(bf16_np(y), oracle.gemv(xq[0], np.float32(1e-2), q, ws, 1))
        ex = np.sort(rng.integers(0, 2, M)).astype(np.int32)
        off, ts, mt = M_.segments(cuda(ex), 2, 128)
        xp = cuda(np.concatenate([xq, np.zeros((128, K), np.int8)]))
        acc = M_.moe_mm(xp, M, torch.stack([c, c]), torch.stack([b, b]), torch.stack([s, s]), off, ts, mt, N, 0)
        _status_ok(scmx)
        assert np.array_equal(acc.cpu().numpy(), oracle.gemm_i32(xq, q))
    finally:
        S.set_format(F.Format())


@pytest.mark.gpu
@pytest.mark.parametrize("K", [2048, 6144])
def test_gemv_fused_prologue_equals_row_kernel_then_gemv(scmx, oracle, K):
    """The in-kernel prologues (scmx_gemv_pro) against the separate row kernels, bit for bit, for every epilogue and for
    per-slot input rows of the expert form."""
    G, S, F = scmx.sc_decode, scmx.sc_kernels, scmx.sc_format
    rng = np.random.default_rng(K)
    N = 1024
    oc, ob, ows, _ = oracle.quantize(rng.standard_normal((N, K)) * 0.02)
    c, b, s = F.to_device(oc, ob, ows)
    x = to_bf16_cuda(oracle.bf16_round((rng.standard_normal((1, K)) * rng.lognormal(0, 1, K)).astype(np.float32)))
    nw = to_bf16_cuda(oracle.bf16_round(rng.lognormal(0, 0.3, K).astype(np.float32)))
    res = to_bf16_cuda(oracle.bf16_round(rng.standard_normal(N).astype(np.float32)))
    for pro in (1, 2):
        for epi in (1, 2, 3):
            outs = []
            for fuse in (True, False):
                outs.append(G.gemv(x, c, b, None, s, N, epi, res=res if epi == 2 else None, pro=pro, nw=nw, eps=1e-6, fuse=fuse))
            assert torch.equal(outs[0], outs[1]), (pro, epi)
    # zero row: scale 0, all-zero codes, output exactly the residual
    z = torch.zeros_like(x)
    y = G.gemv(z, c, b, None, s, N, 2, res=res, pro=1, fuse=True)
    assert torch.equal(y, res)
    # expert form with one input row per slot
    E, Ne = 4, 256
    packs = [oracle.quantize(rng.standard_normal((Ne, K)) * 0.02) for _ in range(E)]
    cE, bE, sE = (torch.stack([F.to_device(*p[:3])[i] for p in packs]) for i in range(3))
    xr = to_bf16_cuda(oracle.bf16_round(rng.standard_normal((3, K)).astype(np.float32) * 2))
    e = cuda(np.array([3, 0, 2], np.int32))
    outs = []
    for fuse in (True, False):
        outs.append(G.gemv(xr, cE, bE, None, sE, Ne, 1, eidx=e, xstride=1, pro=1, fuse=fuse))
    assert torch.equal(outs[0], outs[1])


@pytest.mark.parametrize("M,N,K,epi", [(2048, 4096, 2048, 1), (2048, 2048, 6144, 2), (1024, 1344, 1024, 3), (256, 256, 128, 0),
                                       (640, 288, 4096, 1)])
def test_pair_kernel_equals_single_cta_kernel(scmx, M, N, K, epi):
    """Dense GEMMs run on CTA pairs (cta_group::2, 256 x 256 tiles) by default; the single-CTA kernel (128 x 256 tiles) must
    give the same bits for every epilogue, with ragged M and N tails."""
    S = scmx.sc_kernels
    g = torch.Generator(device="cuda").manual_seed(M + N)
    xq = torch.randint(-127, 128, (M, K), dtype=torch.int8, device="cuda", generator=g)
    wq = torch.randint(-96, 97, (N, K), dtype=torch.int8, device="cuda", generator=g)
    xs = torch.rand(M, device="cuda", generator=g) * 1e-3
    ws = torch.rand(N, device="cuda", generator=g) * 1e-3
    res = torch.randn((M, N), device="cuda", generator=g).to(torch.bfloat16)

    def run():
        if epi == 0:
            return S.mm_i8_i32(xq, wq)
        return S.mm_epi(xq, wq, xs, ws, epi, res=res if epi == 2 else None)
    a = run()
    scmx._lib.call("scmx_set_gemm_pair", 0)
    try:
        b = run()
    finally:
        scmx._lib.call("scmx_set_gemm_pair", 1)
    _status_ok(scmx)
    assert torch.equal(a, b)
    if epi == 0:
        assert torch.equal(a, torch._int_mm(xq, wq.t()) if M > 32 and M % 8 == 0 else a)


@pytest.mark.parametrize("M,N,K,epi", [(512, 1024, 2048, 2), (384, 768, 512, 3), (256, 256, 128, 1)])
def test_gemm_with_gather_epilogue_one_rank(scmx, M, N, K, epi):
    """scmx_mm_i8_bcast (the GEMM whose epilogue stores every output line into all ranks' buffers) with a world of one rank, and
    with two output buffers on the same GPU standing in for two ranks: every copy equals the plain GEMM's output."""
    import ctypes
    S, L = scmx.sc_kernels, scmx._lib
    g = torch.Generator(device="cuda").manual_seed(M + K)
    xq = torch.randint(-127, 128, (M, K), dtype=torch.int8, device="cuda", generator=g)
    wq = torch.randint(-96, 97, (N, K), dtype=torch.int8, device="cuda", generator=g)
    xs = torch.rand(M, device="cuda", generator=g) * 1e-3
    ws = torch.rand(N, device="cuda", generator=g) * 1e-3
    res = torch.randn((M, N), device="cuda", generator=g).to(torch.bfloat16)
    ref = S.mm_epi(xq, wq, xs, ws, epi, res=res if epi == 2 else None)
    for world in (1, 2):
        outs = [torch.full_like(ref, -3) for _ in range(world)]
        peers = (ctypes.c_void_p * 8)(*[o.data_ptr() for o in outs], *([None] * (8 - world)))
        L.call("scmx_mm_i8_bcast", L.ptr(xq), L.ptr(wq), M, N, K, epi, L.ptr(xs), L.ptr(ws), L.ptr(res) if epi == 2 else None,
               peers, world, L.ptr(L.status_buffer()), L.stream())
        _status_ok(scmx)
        for o in outs:
            assert torch.equal(o, ref)
    # shapes the CTA-pair kernel does not take are refused, not silently run elsewhere
    out = torch.empty_like(ref)
    peers = (ctypes.c_void_p * 8)(out.data_ptr(), *([None] * 7))
    assert L.lib().scmx_mm_i8_bcast(L.ptr(xq), L.ptr(wq), 128, N, K, 1, L.ptr(xs), L.ptr(ws), None, peers, 1,
                                    L.ptr(L.status_buffer()), L.stream()) == -5
