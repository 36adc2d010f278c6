"""GPU parity: activation quantization, RMSNorm + quant, SwiGLU, residual epilogue, MoE combine, routing."""
import numpy as np
import pytest
import torch

from helpers import bf16_np, cuda, llm_acts, to_bf16_cuda

pytestmark = pytest.mark.gpu


def test_act_quant_reference_vectors(scmx, golden):
    xq, xs = scmx.sc_kernels.act_quant(to_bf16_cuda(golden["actq_x"]))
    assert xq.shape == (128, 1024) and xs.shape == (128,)
    assert np.array_equal(xq[:40].cpu().numpy(), golden["actq_q"])
    assert np.array_equal(xs[:40].cpu().numpy(), golden["actq_s"])
    assert not xq[40:].any() and not xs[40:].any()


@pytest.mark.parametrize("M,K", [(200, 2048), (1, 2048), (127, 6144), (512, 2048), (3, 2560), (16, 64)])
def test_act_quant_against_oracle(scmx, oracle, M, K):
    rng = np.random.default_rng(M + K)
    x = llm_acts(rng, M, K, oracle)
    x[0] = 0
    xq, xs = scmx.sc_kernels.act_quant(to_bf16_cuda(x))
    oq, os_ = oracle.act_quant(x, oracle.pad_rows(M))
    assert np.array_equal(xq.cpu().numpy(), oq) and np.array_equal(xs.cpu().numpy(), os_)


def test_act_quant_empty(scmx):
    xq, xs = scmx.sc_kernels.act_quant(torch.zeros((0, 256), dtype=torch.bfloat16, device="cuda"), 128)
    assert xq.shape == (128, 256) and not xq.any() and not xs.any()


@pytest.mark.parametrize("M,K", [(200, 2048), (5, 4096), (64, 1024)])
def test_rmsnorm_quant_against_oracle(scmx, oracle, M, K):
    rng = np.random.default_rng(7)
    x = oracle.bf16_round((rng.standard_normal((M, K)) * rng.lognormal(0, 1, (1, K))).astype(np.float32))
    nw = oracle.bf16_round(rng.lognormal(0, 0.3, K).astype(np.float32))
    xq, xs, xn = scmx.sc_kernels.rmsnorm_quant_n(to_bf16_cuda(x), to_bf16_cuda(nw), 1e-6)
    oq, os_, on = oracle.rmsnorm_quant(x, nw, 1e-6, oracle.pad_rows(M))
    assert np.array_equal(bf16_np(xn), on)
    assert np.array_equal(xq.cpu().numpy(), oq) and np.array_equal(xs.cpu().numpy(), os_)
    xq2, xs2 = scmx.sc_kernels.rmsnorm_quant(to_bf16_cuda(x), to_bf16_cuda(nw), torch.tensor([1e-6], device="cuda"))
    assert torch.equal(xq2, xq) and torch.equal(xs2, xs)


def test_swiglu_exhaustive_over_bf16_gates(scmx, oracle):
    """Every bf16 gate value against random up values (the reference's check 4, e2e/test_sc_kernels.py:80-93).
    The only gate magnitude whose exp sits within 4 float32 ulps of a bf16 rounding boundary is 6.84375; it is allowed
    to differ by the rounding of that one intermediate."""
    rng = np.random.default_rng(0)
    bits = np.arange(65536, dtype=np.uint32).astype(np.uint16)
    g = oracle.bf16_from_bits(bits).copy()
    g[~np.isfinite(g)] = 0
    u = oracle.bf16_round((rng.standard_normal(65536) * 3).astype(np.float32))
    out = bf16_np(scmx.sc_kernels.sc_swiglu(to_bf16_cuda(g), to_bf16_cuda(u)))
    ref = oracle.swiglu_bf16(g, u)
    diff = np.flatnonzero(out != ref)
    assert set(np.abs(g[diff]).tolist()) <= {6.84375}, f"{len(diff)} outputs differ, gates {np.unique(g[diff])[:8]}"


def test_res_epilogue_and_swiglu_quant(scmx, oracle):
    rng = np.random.default_rng(4)
    Mp, N = 256, 1024
    acc = rng.integers(-2 ** 20, 2 ** 20, (Mp, N)).astype(np.int32)
    xs = (np.abs(rng.standard_normal(Mp)) * 1e-3).astype(np.float32)
    ws = (np.abs(rng.standard_normal(N)) * 1e-3).astype(np.float32)
    res = oracle.bf16_round(rng.standard_normal((Mp, N)).astype(np.float32))
    h = scmx.sc_kernels.res_epilogue(cuda(acc), cuda(xs), cuda(ws), to_bf16_cuda(res))
    assert np.array_equal(bf16_np(h), oracle.epilogue(acc, xs, ws, 2, res))
    # swiglu_quant: gate | up halves (not interleaved)
    y = oracle.epilogue(acc, xs, ws, 1)
    a = oracle.swiglu_bf16(y[:, :N // 2], y[:, N // 2:])
    oq, os_ = oracle.act_quant(a)
    xq, xs2 = scmx.sc_kernels.swiglu_quant(cuda(acc), cuda(xs), cuda(ws))
    assert np.array_equal(xq.cpu().numpy(), oq) and np.array_equal(xs2.cpu().numpy(), os_)
    # res_norm_quant = res_epilogue + rmsnorm_quant
    nw = oracle.bf16_round(rng.lognormal(0, 0.3, N).astype(np.float32))
    h2, q2, s2 = scmx.sc_kernels.res_norm_quant(cuda(acc), cuda(xs), cuda(ws), to_bf16_cuda(res), to_bf16_cuda(nw), 1e-6)
    oq2, os2, _ = oracle.rmsnorm_quant(bf16_np(h), nw, 1e-6)
    assert torch.equal(h2, h) and np.array_equal(q2.cpu().numpy(), oq2) and np.array_equal(s2.cpu().numpy(), os2)


@pytest.mark.parametrize("E,M,k", [(8, 300, 2), (64, 1000, 8), (128, 257, 8), (3, 1, 1), (64, 4096, 8), (1000, 1025, 8), (16, 8191, 2)])
def test_route_sort_contract(scmx, oracle, E, M, k):
    rng = np.random.default_rng(E + M)
    inds = np.stack([rng.permutation(E)[:k] for _ in range(M)]).astype(np.int32)
    if E >= 8:
        inds[inds == 3] = 2          # expert 3 empty (duplicates within a token do not matter to the sort)
        inds[inds == E - 1] = 0      # last expert empty
    pos, tok, es, off, ts, maxt = scmx.sc_moe.route_sort(cuda(inds), E, 128)
    assert maxt == -(-M * k // 128) + E
    assert oracle.check_route(inds, E, 128, pos.cpu().numpy(), tok.cpu().numpy(), es.cpu().numpy(), off.cpu().numpy(),
                              ts.cpu().numpy())
    off2, ts2, _ = scmx.sc_moe.segments(es, E, 128)
    assert torch.equal(off2, off) and torch.equal(ts2, ts)


def test_router_topk(scmx, oracle):
    rng = np.random.default_rng(9)
    lg = rng.standard_normal((500, 64)).astype(np.float32)
    inds, scores = scmx.sc_moe.router_topk(cuda(lg), 8)
    oi, osc = oracle.softmax_topk(lg, 8)
    assert np.array_equal(inds.cpu().numpy(), oi)
    np.testing.assert_allclose(bf16_np(scores), oracle.bf16_round(osc), rtol=2 ** -7, atol=0)   # within 1 bf16 ulp


def test_moe_combine_against_oracle(scmx, oracle):
    rng = np.random.default_rng(6)
    M, Mp, k, K = 200, 256, 8, 2048
    R = M * k
    y = oracle.bf16_round(rng.standard_normal((R, K)).astype(np.float32))
    sc = oracle.bf16_round(np.abs(rng.standard_normal((M, k)) * 0.2).astype(np.float32))
    res = oracle.bf16_round(rng.standard_normal((Mp, K)).astype(np.float32))
    res[M:] = 0
    nw = oracle.bf16_round(rng.lognormal(0, 0.3, K).astype(np.float32))
    pos = rng.permutation(R).astype(np.int32)
    h, xq, xs = scmx.sc_moe.moe_combine(to_bf16_cuda(y), cuda(pos), to_bf16_cuda(sc), to_bf16_cuda(res), to_bf16_cuda(nw),
                                        1e-5, M)
    oh = oracle.moe_combine(y, pos, sc, res, M)
    assert np.array_equal(bf16_np(h), oh)
    oq, os_, _ = oracle.rmsnorm_quant(oh, nw, 1e-5)
    assert np.array_equal(xq.cpu().numpy(), oq) and np.array_equal(xs.cpu().numpy(), os_)
    h2, _, _ = scmx.sc_moe.moe_combine(to_bf16_cuda(y), cuda(pos), to_bf16_cuda(sc), to_bf16_cuda(res), to_bf16_cuda(nw),
                                       1e-5, M, quant=False)
    assert torch.equal(h2, h)


def test_gather_rows(scmx):
    rng = np.random.default_rng(1)
    xq = rng.integers(-127, 128, (50, 256)).astype(np.int8)
    xs = rng.standard_normal(50).astype(np.float32)
    tok = rng.integers(0, 50, 300 + 128).astype(np.int32)
    dq, ds = scmx.sc_moe.gather_rows(cuda(xq), cuda(xs), cuda(tok), 300)
    assert np.array_equal(dq.cpu().numpy(), xq[tok]) and np.array_equal(ds.cpu().numpy(), xs[tok[:300]])


@pytest.mark.gpu
@pytest.mark.parametrize("M,K", [(5, 96), (130, 2048), (3, 6144), (1, 8192)])
def test_rot_quant_matches_oracle(scmx, oracle, M, K):
    rng = np.random.default_rng(M + K)
    x = oracle.bf16_round((rng.standard_normal((M, K)) * rng.lognormal(0, 1, (1, K))).astype(np.float32))
    x[0, :32] = 0                                         # a zero block
    signs = oracle.rot_signs(K)
    Mp = M + 3
    xq, xs = scmx.sc_kernels.rot_quant(to_bf16_cuda(x), scmx.sc_kernels.rot_signs(K), Mp)
    oq, os_ = oracle.rot_quant(x, signs, Mp)
    assert np.array_equal(xq.cpu().numpy(), oq) and np.array_equal(xs.cpu().numpy(), os_)
    assert not xq[M:].any() and not xs[M:].any()
    z, zs = scmx.sc_kernels.rot_quant(torch.zeros((2, K), dtype=torch.bfloat16, device="cuda"), scmx.sc_kernels.rot_signs(K), 2)
    assert not z.any() and not zs.any()
