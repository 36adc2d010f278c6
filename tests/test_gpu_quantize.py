"""GPU parity: the CUDA quantizer / packer / unpack against the reference vectors and the oracle (bit-exact)."""
import numpy as np
import pytest
import torch

from helpers import cuda, llm_weights, sha

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("tag", ["a", "b", "c", "f64"])
def test_quantize_reference_vectors(scmx, golden, tag):
    w = golden[f"quantize_{tag}_w"]
    codes, bc, ws, qw = scmx.sc_format.quantize(w)
    assert codes.dtype == np.uint32 and bc.dtype == np.uint8 and ws.dtype == np.float32 and qw.dtype == np.int8
    assert np.array_equal(codes, golden[f"quantize_{tag}_codes"])
    assert np.array_equal(bc, golden[f"quantize_{tag}_bcodes"])
    assert np.array_equal(ws, golden[f"quantize_{tag}_wscale"])
    assert np.array_equal(qw, golden[f"quantize_{tag}_qw"])


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64, torch.bfloat16])
@pytest.mark.parametrize("sigma", [0.3, 2.0])
def test_quantize_against_oracle(scmx, oracle, dtype, sigma):
    rng = np.random.default_rng(11)
    w = llm_weights(rng, 192, 2048, sigma)
    w[5, 128:160] = 0
    w[9] = 0
    wt = cuda(w).to(dtype)
    codes, bc, ws, qw, rexp = scmx.sc_format.quantize_device(wt)
    r = oracle.quantize_rows(wt.double().cpu().numpy())
    oc, ob, ows, oqw = oracle.quantize(wt.double().cpu().numpy())
    assert np.array_equal(codes.cpu().numpy().view(np.uint32), oc)
    assert np.array_equal(bc.cpu().numpy(), ob)
    assert np.array_equal(ws.cpu().numpy(), ows)
    assert np.array_equal(qw.cpu().numpy(), oqw)
    assert np.array_equal(rexp.cpu().numpy(), r["elo"])        # row exponents E_lo
    # spread constraint and exact embedding (size-independent properties)
    assert int(r["shift"].max()) <= 3 and np.abs(qw.cpu().numpy().astype(np.int32)).max() <= 96


def test_quantize_headline_layer_digests(scmx, digests):
    """The 6144 x 2048 weight matrix of the single-layer configuration: digests of the packed outputs equal the ones
    recorded from the reference's quantizer."""
    r0 = np.random.default_rng(0)
    W = (r0.standard_normal((6144, 2048)) * 0.02).astype(np.float32)
    if sha(W) != digests["W"]:
        pytest.skip("NumPy's generator stream differs from the one the digests were recorded with")
    codes, bc, ws, qw = scmx.sc_format.quantize(W)
    assert sha(codes) == digests["codes"] and sha(bc) == digests["bcodes"] and sha(ws) == digests["wscale"]


def test_unpack_equals_decode(scmx, oracle, golden):
    S, F = scmx.sc_kernels, scmx.sc_format
    for tag in "abc":
        qw = golden[f"quantize_{tag}_qw"]
        c, b, s = F.to_device(golden[f"quantize_{tag}_codes"], golden[f"quantize_{tag}_bcodes"], golden[f"quantize_{tag}_wscale"])
        assert np.array_equal(S.unpack_i8(c, b, *qw.shape).cpu().numpy(), qw)


FORMATS = [dict(), dict(block=16), dict(block=32, mult=(1, 2, 3, 4)),
           dict(block=16, mult=(1, 2, 3, 4, 5, 6, 8, 10), bc_bits=4),
           dict(block=32, code_mag=(0, 1, 2, 3, 4, 5, 6, 7), mult=(1, 3, 9, 15)),
           dict(block=8, mult=tuple(range(1, 11)), bc_bits=4), dict(block=64, mult=(1, 2), bc_bits=1)]


@pytest.mark.parametrize("kw", FORMATS)
def test_unpack_generic_formats_random_codes(scmx, oracle, kw):
    """Random codes (including negative zero) and block codes of other formats (e2e/test_formats.py:16-35)."""
    S, F = scmx.sc_kernels, scmx.sc_format
    fmt = F.Format(**kw)
    rng = np.random.default_rng(0)
    N, K = 96, 2048
    c4 = rng.integers(0, 16, (N, K)).astype(np.uint8)
    bcode = rng.integers(0, len(fmt.mult), (N, K // fmt.block)).astype(np.uint8)
    codes, bc, ws = F.pack_rows(c4, bcode, np.ones(N), fmt)
    q = oracle.decode(codes, bc, N, K, oracle.Format(fmt.block, fmt.code_mag, fmt.mult, fmt.bc_bits))
    S.set_format(fmt)
    try:
        c, b, _ = F.to_device(codes, bc, ws)
        assert np.array_equal(S.unpack_i8(c, b, N, K).cpu().numpy(), q)
    finally:
        S.set_format(F.Format())


@pytest.mark.parametrize("tag", ["b16pow2", "b16m10", "b32m8", "i4b16"])
def test_family_quantizer_reference_vectors(scmx, golden, tag):
    F = scmx.sc_format
    f = golden[f"family_{tag}_fmt"]
    fmt = F.Format(block=int(f[0]), code_mag=tuple(int(v) for v in f[2:10]), mult=tuple(int(v) for v in f[10:]), bc_bits=int(f[1]))
    codes, bc, ws, qw = F.family_quantize_device(cuda(golden["family_w"]), fmt)
    assert np.array_equal(qw.cpu().numpy(), golden[f"family_{tag}_qi"])
    assert np.array_equal(ws.cpu().numpy(), golden[f"family_{tag}_base"])
    assert np.array_equal(codes.cpu().numpy().view(np.uint32), golden[f"family_{tag}_codes"])
    assert np.array_equal(bc.cpu().numpy(), golden[f"family_{tag}_bcodes"])


def test_family_quantizer_against_oracle_config5_shape(scmx, oracle):
    """16-wide blocks, 2^shift multipliers, a [768, 2048] expert matrix of the large-MoE configuration (sampled rows)."""
    F = scmx.sc_format
    rng = np.random.default_rng(2)
    w = llm_weights(rng, 96, 2048, 0.5)
    fmt = F.Format(block=16)
    codes, bc, ws, qw = F.family_quantize_device(cuda(w), fmt)
    oc, ob, ows, oq = oracle.family_pack(w, oracle.Format(block=16))
    assert np.array_equal(qw.cpu().numpy(), oq) and np.array_equal(ws.cpu().numpy(), ows)
    assert np.array_equal(codes.cpu().numpy().view(np.uint32), oc) and np.array_equal(bc.cpu().numpy(), ob)
