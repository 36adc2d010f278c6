"""CPU: the oracle against the fixtures produced by the reference's own NumPy code, and the exactness properties
the reference's self-tests assert (sim/mx_int8.py:194-209, sim/formats.py:136-148, e2e/sc_format.py:114-127)."""
import numpy as np
import pytest


@pytest.mark.parametrize("tag", ["a", "b", "c", "f64"])
def test_quantize_matches_reference(oracle, golden, tag):
    w = golden[f"quantize_{tag}_w"]
    codes, bc, ws, qw = oracle.quantize(w)
    assert np.array_equal(codes, golden[f"quantize_{tag}_codes"])
    assert np.array_equal(bc, golden[f"quantize_{tag}_bcodes"])
    assert np.array_equal(ws, golden[f"quantize_{tag}_wscale"])
    assert np.array_equal(qw, golden[f"quantize_{tag}_qw"])
    assert np.array_equal(oracle.decode(codes, bc, *w.shape), qw)


def test_constrained_exponents_match_reference(oracle, golden):
    for tag in "abc":
        w = golden[f"quantize_{tag}_w"].astype(np.float64)
        e = oracle.constrain_spread(oracle.block_exponents_search(w))
        assert np.array_equal(e.astype(np.int32), golden[f"quantize_{tag}_e"])
        assert (e.max(1) - e.min(1)).max() <= 3


def test_int8_embedding_is_exact(oracle):
    """q * 2^(E_lo-1) reproduces the MXFP4 fake-quantized weights and the INT8 GEMM equals x @ Wq^T (self_test)."""
    rng = np.random.default_rng(0)
    w = rng.standard_normal((64, 1024)) * rng.lognormal(0, 1.0, (1, 1024))
    r = oracle.quantize_rows(w)
    e = oracle.constrain_spread(oracle.block_exponents_search(w))
    b = w.reshape(64, -1, 32)
    t = b / np.exp2(e)[..., None]
    v = np.sign(t) * np.array([0, .5, 1, 1.5, 2, 3, 4, 6])[oracle.e2m1_index(np.abs(t))]
    wq = (v * np.exp2(e)[..., None]).reshape(w.shape)
    assert np.array_equal(r["qw"].astype(np.float64) * r["wscale"].astype(np.float64)[:, None], wq)
    assert np.abs(r["qw"].astype(np.int32)).max() <= 96
    x = rng.integers(-127, 128, (8, 1024))
    acc = oracle.gemm_i32(x, r["qw"])
    assert np.array_equal(acc.astype(np.float64) * r["wscale"].astype(np.float64)[None], x.astype(np.float64) @ wq.T)


@pytest.mark.parametrize("tag", ["b16pow2", "b16m10", "b32m8", "i4b16"])
def test_family_matches_reference(oracle, golden, tag):
    f = golden[f"family_{tag}_fmt"]
    fmt = oracle.Format(int(f[0]), tuple(int(v) for v in f[2:10]), tuple(int(v) for v in f[10:]), int(f[1]))
    codes, bc, ws, qi = oracle.family_pack(golden["family_w"], fmt)
    assert np.array_equal(qi, golden[f"family_{tag}_qi"])
    assert np.array_equal(ws, golden[f"family_{tag}_base"])
    assert np.array_equal(codes, golden[f"family_{tag}_codes"])
    assert np.array_equal(bc, golden[f"family_{tag}_bcodes"])


def test_generic_pack_decode(oracle, golden):
    fmt = oracle.Format(block=16, mult=(1, 2, 3, 4, 5, 6, 8, 10), bc_bits=4)
    cc, bb, _ = oracle.pack_rows(golden["generic_code4"], golden["generic_bcode"], np.ones(8), fmt)
    assert np.array_equal(cc, golden["generic_codes"]) and np.array_equal(bb, golden["generic_bcodes"])
    assert np.array_equal(oracle.decode(cc, bb, 8, 256, fmt), golden["generic_q"])


def test_act_quant_matches_reference(oracle, golden):
    q, s = oracle.act_quant(golden["actq_x"])
    assert np.array_equal(q, golden["actq_q"]) and np.array_equal(s, golden["actq_s"])
    qp, sp = oracle.act_quant(golden["actq_x"], 128)
    assert np.array_equal(qp[:40], q) and not qp[40:].any() and not sp[40:].any()


def test_interleave_matches_reference(oracle, golden):
    assert np.array_equal(oracle.interleave_gate_up(768), golden["perm_768"])


def test_route_sort_contract(oracle):
    rng = np.random.default_rng(3)
    inds = np.stack([rng.permutation(8)[:2] for _ in range(300)]).astype(np.int32)
    out = oracle.route_sort(inds, 8, 128)
    assert oracle.check_route(inds, 8, 128, *out[:5])
    inds2 = np.where(inds == 7, 0, inds)      # expert 7 empty (duplicates per token are fine for the sort)
    out2 = oracle.route_sort(inds2, 8, 128)
    assert oracle.check_route(inds2, 8, 128, *out2[:5]) and out2[3][8] - out2[3][7] == 0


def test_swiglu_exp_rounding_is_robust(oracle):
    """For every non-negative finite bf16 g except one (g = 6.84375, bits 0x40db), exp(g) is at least 4 float32 ulps
    away from a bf16 rounding boundary (or overflows), so any float32 exp accurate to a couple of ulps gives the same
    bf16 value as the oracle's correctly rounded one: the GPU epilogue can use expf and still match bit for bit,
    and the exhaustive GPU check singles out that one input."""
    bits = np.arange(0, 0x7F80, dtype=np.uint16)
    g = oracle.bf16_from_bits(bits).astype(np.float64)
    with np.errstate(over="ignore"):
        e = np.exp(g)
    fin = e < 3.3e38
    u = e[fin].astype(np.float32).view(np.uint32)
    dist = np.abs((u & np.uint32(0xFFFF)).astype(np.int64) - 0x8000)   # f32 ulps to the bf16 midpoint
    close = bits[fin][dist < 4]
    assert close.tolist() == [0x40DB]


def test_moe_combine_order(oracle):
    rng = np.random.default_rng(5)
    M, k, K = 5, 4, 16
    y = oracle.bf16_round(rng.standard_normal((M * k, K)).astype(np.float32))
    sc = oracle.bf16_round(np.abs(rng.standard_normal((M, k))).astype(np.float32))
    res = oracle.bf16_round(rng.standard_normal((8, K)).astype(np.float32))
    pos = rng.permutation(M * k).astype(np.int32)
    h = oracle.moe_combine(y, pos, sc, res, M)
    t = 2
    acc = np.zeros(K, np.float32)
    for j in range(k):
        acc = oracle.bf16_round(oracle.bf16_round(y[pos[t * k + j]] * sc[t, j]) + acc)
    assert np.array_equal(h[t], oracle.bf16_round(res[t] + acc)) and np.array_equal(h[M:], res[M:])


def test_rot_quant_is_the_sign_flipped_block_hadamard_transform(oracle):
    """The butterfly order restated from e2e/sc_kernels.py:234-275 against the definition: y = H32 (x * signs) / sqrt(32) per
    32-wide block in float64, rounded to bf16, then per-token INT8 (a float32 rounding of a sum may move a code by one)."""
    rng = np.random.default_rng(11)
    M, K = 7, 256
    x = oracle.bf16_round((rng.standard_normal((M, K)) * rng.lognormal(0, 1, (1, K))).astype(np.float32))
    signs = oracle.rot_signs(K)
    assert set(np.unique(signs)) == {-1.0, 1.0} and np.array_equal(signs[:8], np.random.default_rng(0).choice([-1.0, 1.0], size=K)[:8])
    H = np.array([[1.0]])
    while H.shape[0] < 32:
        H = np.block([[H, H], [H, -H]])
    y = ((x.astype(np.float64) * signs).reshape(M, K // 32, 32) @ H.T / np.sqrt(32)).reshape(M, K)
    want_q, want_s = oracle.act_quant(oracle.bf16_round(y.astype(np.float32)), M)
    got_q, got_s = oracle.rot_quant(x, signs, M)
    assert np.abs(got_q.astype(int) - want_q.astype(int)).max() <= 1
    assert (got_q != want_q).mean() < 0.01 and np.allclose(got_s, want_s, rtol=1e-2)


def test_pack_from_values_and_exponents(oracle, golden, scmx):
    """pack_ve of the reference (e2e/gptq_pack.py:29-47) on values moved to neighbouring levels: the oracle's restatement and
    the product's host-side helper reproduce its codes, shifts, row scales and INT8 values."""
    v, e = golden["packve_v"], golden["packve_e"]
    codes, shifts, ws, qw = oracle.pack_values(v, e)
    assert np.array_equal(codes, golden["packve_codes"]) and np.array_equal(shifts, golden["packve_shifts"])
    assert np.array_equal(ws, golden["packve_wscale"]) and np.array_equal(qw, golden["packve_qw"])
    F = scmx.sc_format
    c2, b2, w2, q2 = F.pack_values(v, e)
    want = F.from_shift_layout(golden["packve_codes"], golden["packve_shifts"], golden["packve_wscale"])
    assert np.array_equal(c2, want[0]) and np.array_equal(b2, want[1]) and np.array_equal(w2, want[2])
    assert np.array_equal(q2, golden["packve_qw"])
    # an all-zero block may carry no exponent; anything else there, or an off-grid value, is refused
    e2 = e.copy()
    v2 = v.copy()
    v2[0, 0] = 0
    e2[0, 0] = -np.inf
    c3, b3, w3, q3 = F.pack_values(v2, e2)
    assert not q3[0, :32].any() and np.array_equal(q3[1:], golden["packve_qw"][1:])
    v2[0, 0, 0] = 1.0
    with pytest.raises(ValueError):
        F.pack_values(v2, e2)
    v4 = v.copy()
    v4[0, 0, 0] = 0.75
    with pytest.raises(ValueError):
        F.pack_values(v4, e)
