"""Generates tests/golden/*.npz by running the REFERENCE's own NumPy code (shinyoungkang1/mxfp4-int8-m5).

Run where the reference checkout is available:   python tests/golden/make_golden.py /path/to/reference
The fixtures travel with the repository; the tests never import the reference.

What is recorded (all inputs are stored as float32/int arrays so that no RNG stream has to be reproduced):
  quantize_*    sc_format.quantize(w)  (e2e/sc_format.py:105 -> sim/make_testcase.py:26 -> sim/mx_int8.py)
  family_*      formats.quantize(w, Fmt) + pack_format.pack_parts  (sim/formats.py:64, e2e/pack_format.py:53)
  generic_*     sc_format.pack_rows / decode_numpy on random codes of a non-default Format (e2e/sc_format.py:66,83)
  actq_*        quant_ref, the float32 activation-quant recipe (e2e/test_sc_kernels.py:21-26; the function's source
                is extracted from the file because the module imports MLX at the top)
  perm_*        interleave_gate_up (e2e/sc_kernels.py:520-524; extracted the same way)
  packve_*      gptq_pack.pack_ve: packing from (E2M1 values, block exponents) instead of weights, on values moved to
                neighbouring levels the way a GPTQ rounding would (e2e/gptq_pack.py:29-47)
  config1       sha256 digests of the full 6144x2048 / 512x2048 case of the headline single-layer configuration
"""
import ast
import hashlib
import os
import sys

import numpy as np

OUT = os.path.dirname(os.path.abspath(__file__))


def _extract(path, name):
    """Compile one top-level function of a reference file without importing the module."""
    src = open(path).read()
    for node in ast.parse(src).body:
        if isinstance(node, ast.FunctionDef) and node.name == name:
            ns = {"np": np}
            exec(compile(ast.Module([node], []), path, "exec"), ns)
            return ns[name]
    raise KeyError(name)


def sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()[:16]


def main(ref):
    sys.path.insert(0, os.path.join(ref, "sim"))
    sys.path.insert(0, os.path.join(ref, "e2e"))
    import formats
    import mx_int8
    import sc_format
    import pack_format

    mx_int8.self_test()
    formats.self_test()
    sc_format._self_test()

    rng = np.random.default_rng(1234)
    g = {}

    # ---- SC-MXFP4 quantizer: LLM-like, heavy column spread (constraint binds), planted zero / tiny blocks, zero row
    def stress(n, k, sigma):
        w = (rng.standard_normal((n, k)) * 0.02 * rng.lognormal(0, sigma, (1, k))).astype(np.float32)
        w[1, 32:64] = 0                       # zero block
        w[2] = 0                              # zero row
        w[3, :32] *= np.float32(2.0 ** -8)    # block far below the row maximum
        w[4, 64:96] = np.float32(0.75) * np.float32(2.0 ** -6)   # exact E2M1 rounding ties (0.75 = mid of .5, 1)
        w[5, ::2] = 0
        return w
    for tag, (n, k, sigma) in dict(a=(64, 512, 0.3), b=(48, 1024, 1.0), c=(16, 2048, 2.0)).items():
        w = stress(n, k, sigma)
        codes, bc, ws, qw = sc_format.quantize(w)
        e = mx_int8.constrain_spread(w.astype(np.float64), mx_int8.block_exponents(w.astype(np.float64), "search"))
        g[f"quantize_{tag}_w"] = w
        g[f"quantize_{tag}_codes"], g[f"quantize_{tag}_bcodes"] = codes, bc
        g[f"quantize_{tag}_wscale"], g[f"quantize_{tag}_qw"] = ws, qw
        g[f"quantize_{tag}_e"] = e.astype(np.int32)
        assert np.array_equal(sc_format.decode_numpy(codes, bc, n, k), qw)
    # float64-origin input (not float32 representable)
    w64 = rng.standard_normal((8, 256)) * rng.lognormal(0, 1.0, (1, 256))
    codes, bc, ws, qw = sc_format.quantize(w64)
    g["quantize_f64_w"] = w64
    g["quantize_f64_codes"], g["quantize_f64_bcodes"], g["quantize_f64_wscale"], g["quantize_f64_qw"] = codes, bc, ws, qw

    # ---- integer-exact family (config 5's 16-wide blocks)
    wf = (rng.standard_normal((24, 512)) * 0.02 * rng.lognormal(0, 0.5, (1, 512))).astype(np.float32)
    wf[3] = 0
    g["family_w"] = wf
    for tag, name in dict(b16pow2="e2m1/B16/pow2", b16m10="e2m1/B16/M1..10", b32m8="e2m1/B32/M1..8",
                          i4b16="int4/B16/M1..16").items():
        f = formats.FORMATS[name]
        wq, qi, base, scales = formats.quantize(wf, f)
        fmt = pack_format.sc_format_of(name)
        codes, bc, ws, st = pack_format.pack_parts(wq, qi, base, scales, fmt)
        assert st["exact_q"] and st["exact_w"], (name, st)
        g[f"family_{tag}_qi"], g[f"family_{tag}_base"] = qi, base
        g[f"family_{tag}_codes"], g[f"family_{tag}_bcodes"], g[f"family_{tag}_wscale"] = codes, bc, ws
        g[f"family_{tag}_fmt"] = np.array([fmt.block, fmt.bc_bits, *fmt.code_mag, *fmt.mult], np.int32)

    # ---- generic pack/decode on random codes
    fmt = sc_format.Format(block=16, mult=(1, 2, 3, 4, 5, 6, 8, 10), bc_bits=4)
    c4 = rng.integers(0, 16, (8, 256)).astype(np.uint8)
    b = rng.integers(0, 8, (8, 16)).astype(np.uint8)
    cc, bb, _ = sc_format.pack_rows(c4, b, np.ones(8), fmt)
    g["generic_code4"], g["generic_bcode"], g["generic_codes"], g["generic_bcodes"] = c4, b, cc, bb
    g["generic_q"] = sc_format.decode_numpy(cc, bb, 8, 256, fmt)

    # ---- activation quant recipe
    quant_ref = _extract(os.path.join(ref, "e2e", "test_sc_kernels.py"), "quant_ref")
    import ml_dtypes
    x = rng.standard_normal((40, 1024)) * rng.lognormal(0, 0.5, (1, 1024))
    x[:, rng.choice(1024, 8, replace=False)] *= 20
    x[7] = 0
    x = x.astype(ml_dtypes.bfloat16).astype(np.float32)
    q, s = quant_ref(x)
    g["actq_x"], g["actq_q"], g["actq_s"] = x, q, s

    perm = _extract(os.path.join(ref, "e2e", "sc_kernels.py"), "interleave_gate_up")
    g["perm_768"] = perm(768).astype(np.int32)

    # ---- packing from values and exponents (GPTQ-rounded tensors keep the exponents of the unquantized weights)
    import gptq_pack
    r2 = np.random.default_rng(77)
    w = (r2.standard_normal((8, 256)) * 0.02 * r2.lognormal(0, 1.0, (1, 256))).astype(np.float64)
    w[1, 32:64] = 0
    e = mx_int8.constrain_spread(w, mx_int8.block_exponents(w, "search"))
    v = mx_int8.blocks(mx_int8.dequant_mx(w, e)[0]) / 2.0 ** e[..., None]          # round-to-nearest E2M1 values
    lv = mx_int8.E2M1
    idx = np.searchsorted(lv, np.abs(v))
    move = r2.random(v.shape) < 0.15                                                 # some weights go to a neighbouring level
    idx2 = np.clip(idx + np.where(move, r2.choice([-1, 1], size=v.shape), 0), 0, 7)
    sgn = np.where(v < 0, -1.0, np.where(v > 0, 1.0, r2.choice([-1.0, 1.0], size=v.shape)))
    v2 = sgn * lv[idx2]
    packed, shifts, wscale, qw = gptq_pack.pack_ve(v2, e)
    g["packve_v"], g["packve_e"] = v2, e
    g["packve_codes"], g["packve_shifts"] = packed.reshape(-1).view(np.uint32).copy(), shifts
    g["packve_wscale"], g["packve_qw"] = wscale, qw

    np.savez_compressed(os.path.join(OUT, "reference_vectors.npz"), **g)

    # ---- headline single-layer configuration, digests only
    r0 = np.random.default_rng(0)
    W = (r0.standard_normal((6144, 2048)) * 0.02).astype(np.float32)
    X = r0.standard_normal((512, 2048))
    cols = r0.choice(2048, 8, replace=False)
    X[:, cols] *= 20
    X = X.astype(ml_dtypes.bfloat16).astype(np.float32)
    codes, bc, ws, qw = sc_format.quantize(W)
    xq, xs = quant_ref(X)
    acc = (xq.astype(np.float64) @ qw.astype(np.float64).T).astype(np.int64).astype(np.int32)
    dig = dict(W=sha(W), X=sha(X), codes=sha(codes), bcodes=sha(bc), wscale=sha(ws), xq=sha(xq), xs=sha(xs),
               acc=sha(acc))
    with open(os.path.join(OUT, "config1_digests.txt"), "w") as fh:
        for k, v in dig.items():
            fh.write(f"{k} {v}\n")
    print(dig)
    print("wrote", sorted(g), "->", OUT)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/make_golden.py /path/to/reference")
    main(sys.argv[1])
