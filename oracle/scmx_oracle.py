"""CPU restatement (NumPy) of the reference's SC-MXFP4 W4A8 hot path.  TEST INFRASTRUCTURE ONLY.

This file is the checker the CUDA kernels are compared against.  It is imported by the test-suite, by the
smoke check and by the CPU-baseline / reference legs of the benchmark, and by nothing else: the product package
never imports it and has no CPU fallback.

Every function cites the reference file:line (paths inside shinyoungkang1/mxfp4-int8-m5) whose arithmetic it
restates.  Parity status: the quantizer / packer / INT32 / activation-quant / routing parts are PINNED against
outputs of the reference's own NumPy code (tests/golden/*.npz, written by tests/golden/make_golden.py which imports
the reference).  The RMSNorm reduction order and the SwiGLU `exp` rounding of the reference's Metal kernels are
compared by the reference against MLX ops that are not available here: those two are "parity unpinned" and the
outputs that depend on them are held to a relative-L2 tolerance, not bit equality.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

BLOCK = 32
MAX_SPREAD = 3
E2M1_X2 = (0, 1, 2, 3, 4, 6, 8, 12)          # 2 x |E2M1| : e2e/sc_format.py:29
_E2M1 = np.array([0, 0.5, 1, 1.5, 2, 3, 4, 6], np.float64)   # sim/mx_int8.py:19
_E2M1_MIDS = (_E2M1[1:] + _E2M1[:-1]) / 2                     # sim/mx_int8.py:20


# ---------------------------------------------------------------------------------------------------------------
# bf16 helpers (round-to-nearest-even on the float32 bit pattern; the reference's `static_cast<bfloat16_t>`)
# ---------------------------------------------------------------------------------------------------------------

def bf16_round(x):
    """float32 array -> float32 array holding the nearest bfloat16 (ties to even); NaN kept as NaN."""
    x = np.ascontiguousarray(x, np.float32)
    u = x.view(np.uint32)
    r = (u + np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))) & np.uint32(0xFFFF0000)
    out = r.view(np.float32).copy()
    nan = np.isnan(x)
    if nan.any():
        out[nan] = np.nan
    return out


def bf16_bits(x):
    """float32 (already bf16-representable or not) -> uint16 bfloat16 bit patterns, RNE."""
    return (bf16_round(x).view(np.uint32) >> np.uint32(16)).astype(np.uint16)


def bf16_from_bits(b):
    return (np.asarray(b, np.uint16).astype(np.uint32) << np.uint32(16)).view(np.float32)


# ---------------------------------------------------------------------------------------------------------------
# a1-a6: SC-MXFP4 quantizer (float64), sim/mx_int8.py:23-109 and sim/make_testcase.py:26-44
# ---------------------------------------------------------------------------------------------------------------

def e2m1_index(a):
    """Index 0..7 of the E2M1 magnitude nearest to a >= 0, saturating at 6; an exact tie goes to the SMALLER
    magnitude (np.searchsorted side='left' on the midpoints, sim/mx_int8.py:20,25)."""
    a = np.minimum(a, 6.0)
    idx = np.zeros(a.shape, np.int64)
    for m in _E2M1_MIDS:
        idx += a > m
    return idx


def _pairwise32(a):
    """Sum over a last axis of 32 float64 in the order NumPy's pairwise reduction uses for n = 32: eight strided
    partial sums r[j] = ((a[j] + a[j+8]) + a[j+16]) + a[j+24], then ((r0+r1)+(r2+r3)) + ((r4+r5)+(r6+r7)).
    This is what `.sum(-1)` computes in sim/mx_int8.py:36; the CUDA quantizer follows the same order."""
    r = a[..., 0:8] + a[..., 8:16]
    r = r + a[..., 16:24]
    r = r + a[..., 24:32]
    return ((r[..., 0] + r[..., 1]) + (r[..., 2] + r[..., 3])) + ((r[..., 4] + r[..., 5]) + (r[..., 6] + r[..., 7]))


def _block_sq_err(b, e):
    """sum_k (round_e2m1(b / 2^e) * 2^e - b)^2 per block (sim/mx_int8.py:34-36)."""
    s = np.exp2(e)[..., None]
    t = b / s
    v = np.sign(t) * _E2M1[e2m1_index(np.abs(t))]
    d = v * s - b
    return _pairwise32(d * d)


def block_exponents_search(w):
    """Per-32-block exponent: floor(log2 amax) - 2, then e-1 and e+1 tried in that order and kept only when their
    squared error is strictly smaller; all-zero block -> -inf (sim/mx_int8.py:39-65, rule='search')."""
    n, k = w.shape
    assert k % BLOCK == 0
    b = np.asarray(w, np.float64).reshape(n, k // BLOCK, BLOCK)
    amax = np.abs(b).max(-1)
    zero = amax == 0
    with np.errstate(divide="ignore"):
        lg = np.log2(amax)
    lg[zero] = 0
    e = np.floor(lg) - 2
    best, err = e.copy(), _block_sq_err(b, e)
    for d in (-1.0, 1.0):
        ce = _block_sq_err(b, e + d)
        better = ce < err
        best = np.where(better, e + d, best)
        err = np.where(better, ce, err)
    best[zero] = -np.inf
    return best


def constrain_spread(e):
    """Lift every block exponent of a row to at least rowmax - 3; an all-zero row uses rowmax = 0
    (sim/mx_int8.py:68-81 with chunk_blocks=None)."""
    hi = e.max(-1, keepdims=True)
    hi = np.where(np.isfinite(hi), hi, 0.0)
    return np.maximum(e, hi - MAX_SPREAD)


def quantize_rows(w):
    """Full reference pack of an (N, K) matrix: returns dict with
      idx   uint8 [N,K]  E2M1 index 0..7        sign uint8 [N,K]  (v < 0)
      shift uint8 [N,K/32] e_b - E_lo in 0..3    elo  int64 [N]   row exponent E_lo
      qw    int8  [N,K]   = +-2v << shift        wscale f32 [N]   = 2^(E_lo-1)
    (sim/make_testcase.py:26-44 -> sim/mx_int8.py block_exponents/constrain_spread/dequant_mx/embed_int8)."""
    w = np.asarray(w, np.float64)
    n, k = w.shape
    e = constrain_spread(block_exponents_search(w))
    b = w.reshape(n, k // BLOCK, BLOCK)
    t = b / np.exp2(e)[..., None]
    idx = e2m1_index(np.abs(t))
    neg = (t < 0) & (idx > 0)                      # v = sign(t) * E2M1[idx]; v < 0 is false when idx == 0
    elo = e.min(-1)
    shift = (e - elo[:, None]).astype(np.int64)
    assert shift.max() <= MAX_SPREAD
    mag = np.array(E2M1_X2, np.int64)[idx] << shift[..., None]
    qw = np.where(neg, -mag, mag).reshape(n, k).astype(np.int8)
    return dict(idx=idx.reshape(n, k).astype(np.uint8), sign=neg.reshape(n, k).astype(np.uint8),
                shift=shift.astype(np.uint8), elo=elo.astype(np.int64), qw=qw,
                wscale=np.exp2(elo - 1).astype(np.float32))


# ---------------------------------------------------------------------------------------------------------------
# a7: packed storage format, e2e/sc_format.py:26-111
# ---------------------------------------------------------------------------------------------------------------

@dataclass(frozen=True)
class Format:
    """Weight format descriptor (e2e/sc_format.py:26-41): q = +-code_mag[idx] * mult[bcode]."""
    block: int = 32
    code_mag: tuple = E2M1_X2
    mult: tuple = (1, 2, 4, 8)
    bc_bits: int = 2

    def __post_init__(self):
        assert self.block % 8 == 0
        assert self.bc_bits in (1, 2, 4, 8) and len(self.mult) <= 2 ** self.bc_bits
        assert len(self.code_mag) == 8 and max(self.code_mag) * max(self.mult) <= 127

    @property
    def per_byte(self):
        return 8 // self.bc_bits


DEFAULT = Format()


def pack_rows(code4, bcode, wscale, fmt=DEFAULT):
    """code4 uint8 [N,K] (sign<<3|idx), bcode uint8 [N,K/block] -> (codes u32 [N*K/8], bcodes u8 [N,..], wscale f32)
    with element 8j+i of a row in bits 4i..4i+3 of word j and block b in bits bc_bits*(b % per_byte) of byte
    b // per_byte (e2e/sc_format.py:66-80)."""
    n, k = code4.shape
    assert k % fmt.block == 0
    c = code4.astype(np.uint32).reshape(n, k // 8, 8)
    sh = (4 * np.arange(8, dtype=np.uint32))
    codes = np.bitwise_or.reduce(c << sh, axis=-1).astype(np.uint32)
    nb = k // fmt.block
    assert nb % fmt.per_byte == 0 and int(bcode.max(initial=0)) < len(fmt.mult)
    bb = bcode.astype(np.uint32).reshape(n, nb // fmt.per_byte, fmt.per_byte)
    bsh = (fmt.bc_bits * np.arange(fmt.per_byte, dtype=np.uint32))
    bc = np.bitwise_or.reduce(bb << bsh, axis=-1).astype(np.uint8)
    return codes.reshape(-1), bc, np.asarray(wscale, np.float32)


def decode(codes, bc, n, k, fmt=DEFAULT):
    """Packed layout -> INT8 operand q [N,K] (e2e/sc_format.py:83-90)."""
    w = np.asarray(codes, np.uint32).reshape(n, k // 8)
    c = ((w[..., None] >> (4 * np.arange(8, dtype=np.uint32))) & np.uint32(0xF)).reshape(n, k).astype(np.int64)
    bcv = np.asarray(bc, np.uint8).reshape(n, -1).astype(np.uint32)
    b = ((bcv[..., None] >> (fmt.bc_bits * np.arange(fmt.per_byte, dtype=np.uint32)))
         & np.uint32(2 ** fmt.bc_bits - 1)).reshape(n, k // fmt.block).astype(np.int64)
    mag = np.array(fmt.code_mag, np.int64)[c & 7] * np.repeat(np.array(fmt.mult, np.int64)[b], fmt.block, axis=1)
    return np.where(c & 8, -mag, mag).astype(np.int8)


def pack_values(v, e):
    """Packing from E2M1 values v [N, K/32, 32] and block exponents e [N, K/32] instead of from weights: what a rounding
    other than round-to-nearest (GPTQ) produces while keeping the exponents (e2e/gptq_pack.py:29-47, with
    sim/mx_int8.py:92-109 for the INT8 embedding).  Returns (codes uint32 [N*K/8], shifts uint8 [N, K/32] one byte per block,
    wscale f32 [N], qw int8 [N, K]).  A non-finite exponent marks an all-zero block (shift 0); the row exponent is the
    minimum finite one (0 for a row without any)."""
    v = np.asarray(v, np.float64)
    e = np.asarray(e, np.float64)
    n, nb, _ = v.shape
    k = nb * BLOCK
    fin = np.isfinite(e)
    hi = np.where(fin, e, -np.inf).max(-1, keepdims=True)
    hi = np.where(np.isfinite(hi), hi, 0.0)
    lo = np.where(fin, e, hi).min(-1, keepdims=True)
    shift_q = (np.where(fin, e, hi) - lo)                       # the embedding's shift (zero blocks: value 0 anyway)
    q = 2 * v * np.exp2(shift_q)[..., None]
    assert np.abs(q).max() <= 127 and np.all(q == np.round(q)), "not INT8-embeddable"
    shifts = (np.where(fin, e, lo) - lo).astype(np.uint8)       # the stored block codes
    a = np.abs(v.reshape(n, k))
    lv = np.array(E2M1_X2, np.float64) / 2
    idx = np.searchsorted(lv, a).astype(np.uint8)
    assert idx.max() <= 7 and np.array_equal(lv[idx], a), "values are not E2M1 levels"
    code4 = idx | ((v.reshape(n, k) < 0).astype(np.uint8) << 3)
    c = code4.astype(np.uint32).reshape(n, k // 8, 8)
    codes = np.bitwise_or.reduce(c << (4 * np.arange(8, dtype=np.uint32)), axis=-1).astype(np.uint32).reshape(-1)
    return codes, shifts, np.exp2(lo[:, 0] - 1).astype(np.float32), q.reshape(n, k).astype(np.int8)


def quantize(w, fmt=DEFAULT):
    """(N,K) float weights -> (codes, bcodes, wscale, qw) in the published SC-MXFP4 layout
    (e2e/sc_format.py:105-111: make_testcase.pack then from_shift_layout)."""
    assert fmt.block == 32 and tuple(fmt.mult) == (1, 2, 4, 8)
    r = quantize_rows(w)
    code4 = (r["idx"] | (r["sign"] << 3)).astype(np.uint8)
    codes, bc, ws = pack_rows(code4, r["shift"], r["wscale"], fmt)
    return codes, bc, ws, r["qw"]


# ---------------------------------------------------------------------------------------------------------------
# a8: integer-exact format family (float32 math), sim/formats.py:57-107 and e2e/pack_format.py:35-76
# ---------------------------------------------------------------------------------------------------------------

def _pairwise_f32(a):
    """NumPy's pairwise float32 sum over a contiguous last axis of length n (8 <= n <= 128, n % 8 == 0): eight
    strided accumulators then the fixed tree.  Used for both the per-block error sums (n = block) and the per-row
    total (n = number of blocks) of sim/formats.py:90-93."""
    n = a.shape[-1]
    assert n % 8 == 0 and 8 <= n <= 128
    r = a[..., 0:8].astype(np.float32).copy()
    for i in range(8, n, 8):
        r = r + a[..., i:i + 8]
    return ((r[..., 0] + r[..., 1]) + (r[..., 2] + r[..., 3])) + ((r[..., 4] + r[..., 5]) + (r[..., 6] + r[..., 7]))


def family_quantize(w, code_mag, block, mults, base_grid=8):
    """w = base[n] * m[n,b] * (+-C[idx]) with the row base searched over `base_grid` points per octave below the
    largest fitting one and the best multiplier per block by squared error, all in float32
    (sim/formats.py:64-107).  Returns (qi int8 [N,K], base f32 [N], bcode uint8 [N,K/block], code4 uint8 [N,K]).
    Rows need K/block <= 128 blocks for the explicit summation order used here."""
    cb = np.asarray(code_mag, np.float32)
    mids = (cb[1:] + cb[:-1]) / np.float32(2)
    mu = np.asarray(mults, np.float32)
    w = np.asarray(w, np.float32)
    n, k = w.shape
    nb = k // block
    wb = w.reshape(n, nb, block)
    amax = np.abs(wb).max((1, 2))
    amax = np.where(amax == 0, np.float32(1), amax).astype(np.float32)
    base_hi = (amax / (mu[-1] * cb[-1])).astype(np.float32)
    best_err = np.full(n, np.inf, np.float32)
    best_base = base_hi.copy()
    best_m = np.zeros((n, nb), np.int64)

    def rnd(x):
        a = np.minimum(np.abs(x), cb[-1])
        return np.sign(x) * cb[np.searchsorted(mids, a)]

    for j in range(base_grid):
        base = (base_hi * np.float32(2.0 ** (-j / base_grid))).astype(np.float32)
        err = np.empty((n, nb, len(mu)), np.float32)
        for i in range(len(mu)):
            s = (base[:, None, None] * mu[i]).astype(np.float32)
            d = rnd(wb / s) * s - wb
            err[:, :, i] = _pairwise_f32(d * d) if block >= 8 else (d * d).sum(-1)
        mi = err.argmin(-1)
        picked = np.take_along_axis(err, mi[..., None], -1)[..., 0]
        tot = _pairwise_f32(picked) if nb % 8 == 0 and 8 <= nb <= 128 else picked.sum(-1)
        better = tot < best_err
        best_err = np.where(better, tot, best_err)
        best_base = np.where(better, base, best_base)
        best_m = np.where(better[:, None], mi, best_m)
    m = mu[best_m]
    s = (best_base[:, None, None] * m[..., None]).astype(np.float32)
    cv = rnd(wb / s)
    qi = (cv * m[..., None]).reshape(n, k)
    assert np.abs(qi).max() <= 127
    idx = np.searchsorted(cb, np.abs(cv)).reshape(n, k)
    code4 = (idx | ((qi < 0).astype(np.int64) << 3)).astype(np.uint8)
    return qi.astype(np.int8), best_base.astype(np.float32), best_m.astype(np.uint8), code4


def family_pack(w, fmt: Format, base_grid=8):
    """family_quantize + pack_rows: (codes, bcodes, wscale, qi) for a generic Format (e2e/pack_format.py:53-76)."""
    qi, base, bcode, code4 = family_quantize(w, fmt.code_mag, fmt.block, fmt.mult, base_grid)
    codes, bc, ws = pack_rows(code4, bcode, base, fmt)
    return codes, bc, ws, qi


# ---------------------------------------------------------------------------------------------------------------
# a9: per-token INT8 activation quantization, float32 reciprocal recipe
# (e2e/sc_kernels.py:200-229 as pinned by e2e/test_sc_kernels.py:21-26)
# ---------------------------------------------------------------------------------------------------------------

def act_quant(x, Mp=None):
    """x float [M,K] (bf16-representable values in float32) -> (xq int8 [Mp,K], xs f32 [Mp]); rows >= M are zero.
    s = amax / 127, qi = 1 / s (0 if s == 0), q = clip(rint(x * qi), -127, 127), all float32, round-half-even."""
    x = np.asarray(x, np.float32)
    M, K = x.shape
    Mp = M if Mp is None else Mp
    s = (np.abs(x).max(1) / np.float32(127)).astype(np.float32)
    with np.errstate(divide="ignore"):
        qi = np.where(s > 0, np.float32(1) / np.where(s > 0, s, np.float32(1)), np.float32(0)).astype(np.float32)
    q = np.clip(np.rint(x * qi[:, None]), -127, 127).astype(np.int8)
    xq = np.zeros((Mp, K), np.int8)
    xs = np.zeros(Mp, np.float32)
    xq[:M], xs[:M] = q, s
    return xq, xs


def pad_rows(M, tm=128):
    """Rows padded to the GEMM M tile (e2e/sc_kernels.py:476-477)."""
    return -(-M // tm) * tm


# ---------------------------------------------------------------------------------------------------------------
# a11-a13: INT32 GEMM and its epilogues, e2e/sc_kernels.py:53-115,319-328,520-524
# ---------------------------------------------------------------------------------------------------------------

def gemm_i32(xq, wq):
    """acc[m,n] = sum_k xq[m,k] * wq[n,k], exact.  Computed through a float64 BLAS GEMM, exact while
    |acc| < 2^53 (the reference's own method, sim/make_testcase.py:59, e2e/test_sc_kernels.py:47-49)."""
    acc = np.asarray(xq, np.float64) @ np.asarray(wq, np.float64).T
    return acc.astype(np.int64).astype(np.int32)


def interleave_gate_up(F):
    """Row permutation [gate(F); up(F)] -> groups g_2p, g_2p+1, u_2p, u_2p+1 (e2e/sc_kernels.py:520-524)."""
    p = np.arange(F // 2)
    return np.stack([2 * p, 2 * p + 1, F + 2 * p, F + 2 * p + 1], 1).reshape(-1)


def swiglu_bf16(g, u):
    """SiLU(g) * u with every step rounded to bf16 (e2e/sc_kernels.py:319-328):
    e = T(exp|g|), y = T(1 / T(1 + e)), sig = g < 0 ? y : T(1 - y), silu = T(g * sig), out = T(silu * u).
    g, u: float32 arrays holding bf16 values.  exp is taken in float64 and rounded once to float32 then bf16."""
    g = np.asarray(g, np.float32)
    u = np.asarray(u, np.float32)
    with np.errstate(over="ignore"):
        e = bf16_round(np.exp(np.abs(g).astype(np.float64)).astype(np.float32))
        y = bf16_round(np.float32(1) / bf16_round(np.float32(1) + e))
    sig = np.where(g < 0, y, bf16_round(np.float32(1) - y))
    silu = bf16_round(g * sig)
    return bf16_round(silu * u)


def epilogue(acc, xs, ws, epi, res=None):
    """INT32 accumulators -> bf16 outputs (as float32 arrays holding bf16 values), e2e/sc_kernels.py:97-114.
    EPI 1: T((float(acc) * xs[m]) * ws[n]);  EPI 2: T(res + T(...));  EPI 3: SwiGLU of interleaved 4-row groups
    [g0,g1,u0,u1] -> [swiglu(g0,u0), swiglu(g1,u1)], output [M, N/2]."""
    a = (acc.astype(np.float32) * np.asarray(xs, np.float32)[:, None]) * np.asarray(ws, np.float32)[None, :]
    y = bf16_round(a)
    if epi == 1:
        return y
    if epi == 2:
        return bf16_round(np.asarray(res, np.float32) + y)
    assert epi == 3
    M, N = y.shape
    y4 = y.reshape(M, N // 4, 4)
    out = np.empty((M, N // 4, 2), np.float32)
    out[..., 0] = swiglu_bf16(y4[..., 0], y4[..., 2])
    out[..., 1] = swiglu_bf16(y4[..., 1], y4[..., 3])
    return out.reshape(M, N // 2)


# ---------------------------------------------------------------------------------------------------------------
# a14: fused row kernels (RMSNorm + quant, residual epilogue), e2e/sc_kernels.py:123-197
# ---------------------------------------------------------------------------------------------------------------

def rmsnorm_bf16(x, w, eps):
    """w * T(x * rsqrt(mean(x^2) + eps)) with bf16 rounding of x*inv and of the product (e2e/sc_kernels.py:120-143).
    The reference sums x^2 in the thread layout of MLX's rms_norm kernel; here the sum is taken in float64 and
    rounded to float32 (reduction order unpinned, see the module docstring)."""
    x = np.asarray(x, np.float32)
    K = x.shape[1]
    ss = (x.astype(np.float64) ** 2).sum(1).astype(np.float32)
    inv = (np.float32(1) / np.sqrt((ss / np.float32(K) + np.float32(eps)).astype(np.float64))).astype(np.float32)
    return bf16_round(np.asarray(w, np.float32)[None, :] * bf16_round(x * inv[:, None]))


def rmsnorm_quant(x, w, eps, Mp=None):
    """(xq, xs, xn): per-token INT8 of the normalized rows plus the bf16 normalized rows
    (e2e/sc_kernels.py:527-533,619-626)."""
    xn = rmsnorm_bf16(x, w, eps)
    xq, xs = act_quant(xn, Mp)
    out = np.zeros((xq.shape[0], xn.shape[1]), np.float32)
    out[:xn.shape[0]] = xn
    return xq, xs, out


# ---------------------------------------------------------------------------------------------------------------
# rotated-input quantization, e2e/sc_kernels.py:234-275
# ---------------------------------------------------------------------------------------------------------------

def rot_signs(K):
    """e2e/sc_kernels.py:566-569."""
    return np.random.default_rng(0).choice([-1.0, 1.0], size=K).astype(np.float32)


def rot_quant(x, signs, Mp=None):
    """x (bf16 values) [M, K] -> (xq int8 [Mp, K], xs f32 [Mp]).  Per 32-wide block: y = H32 (x * signs) / sqrt(32) with the
    float32 butterfly order of the reference's kernel (element 4t + i of a block belongs to thread t = 0..7: stages over
    i with strides 1 and 2, then over t with strides 1, 2, 4; the side whose index bit is set computes partner - own),
    rounded to bf16; then act_quant."""
    x = np.asarray(x, np.float32)
    M, K = x.shape
    a = (x * np.asarray(signs, np.float32)[None, :]).astype(np.float32).reshape(M, K // 32, 8, 4)   # [.., t, i]
    f = np.float32
    b = np.empty_like(a)
    b[..., 0], b[..., 1] = a[..., 0] + a[..., 1], a[..., 0] - a[..., 1]
    b[..., 2], b[..., 3] = a[..., 2] + a[..., 3], a[..., 2] - a[..., 3]
    a = np.empty_like(b)
    a[..., 0], a[..., 1] = b[..., 0] + b[..., 2], b[..., 1] + b[..., 3]
    a[..., 2], a[..., 3] = b[..., 0] - b[..., 2], b[..., 1] - b[..., 3]
    a = a.astype(f)
    t = np.arange(8)
    for h in (1, 2, 4):
        c = a[:, :, t ^ h, :]
        hi = ((t & h) != 0)[None, None, :, None]
        a = np.where(hi, c - a, a + c).astype(f)
    y = bf16_round((a * f(0.17677669529663687)).astype(f)).reshape(M, K)
    return act_quant(y, Mp)


# ---------------------------------------------------------------------------------------------------------------
# q/k/v epilogue before attention (the callers' glue), e2e/sc_kernels.py:333-423,597-637; rotary step as
# mlx.nn.RoPE(traditional=False) which e2e/fused_qwen3.py:197-203 calls
# ---------------------------------------------------------------------------------------------------------------

def rope_inv_freq(d, base):
    """f32 [d/2]: base^(-2i/d)."""
    i = np.arange(0, d, 2, dtype=np.float64)
    return (1.0 / (float(base) ** (i / d))).astype(np.float32)


def rope_half(x, inv_freq, pos0=0):
    """Half-split rotary embedding of bf16-valued x [h, L, d] at positions pos0 + row: out[i] = x[i] cos - x[i + d/2] sin,
    out[i + d/2] = x[i] sin + x[i + d/2] cos; products and the sum in float32, result rounded to bf16."""
    x = np.asarray(x, np.float32)
    L, d = x.shape[1], x.shape[2]
    ang = (np.arange(pos0, pos0 + L, dtype=np.float32)[:, None] * np.asarray(inv_freq, np.float32)[None, :]).astype(np.float32)
    c = np.cos(ang.astype(np.float64)).astype(np.float32)[None]
    s = np.sin(ang.astype(np.float64)).astype(np.float32)[None]
    x1, x2 = x[..., :d // 2], x[..., d // 2:]
    lo = (x1 * c).astype(np.float32) - (x2 * s).astype(np.float32)
    hi = (x1 * s).astype(np.float32) + (x2 * c).astype(np.float32)
    return bf16_round(np.concatenate([lo, hi], -1))


def qkv_norm(y, qn, kn, eps, L, hq, hk, d, full=False, inv_freq=None, pos0=0):
    """bf16-valued y [>=L, (hq + 2 hk) d] -> q [hq, L, d], k [hk, L, d], v [hk, L, d].  full=False: RMSNorm of every q and
    k head over its d values with weights qn / kn [d] (qkv_headnorm_y, e2e/sc_kernels.py:355-378); full=True: RMSNorm over
    the whole q (hq*d) and k (hk*d) vectors with qn [hq*d], kn [hk*d] (qkv_fullnorm_y, :389-423).  Sum of squares in
    float64 (reduction order unpinned, as for rmsnorm_bf16).  inv_freq: rotary embedding of the normalized q and k."""
    y = np.asarray(y, np.float32)[:L]
    parts = np.split(y, [hq * d, (hq + hk) * d], axis=1)
    out = []
    for x, w, h in ((parts[0], qn, hq), (parts[1], kn, hk)):
        if full:
            n = rmsnorm_bf16(x, w, eps).reshape(L, h, d)
        else:
            n = rmsnorm_bf16(x.reshape(L * h, d), w, eps).reshape(L, h, d)
        n = n.transpose(1, 0, 2)
        out.append(rope_half(n, inv_freq, pos0) if inv_freq is not None else n)
    out.append(parts[2].reshape(L, hk, d).transpose(1, 0, 2))
    return tuple(np.ascontiguousarray(o) for o in out)


def qkv_epilogue_headnorm(acc, xs, ws, qn, kn, eps, L, hq, hk, d, **kw):
    """The same from INT32 accumulators: EPI 1 scaling first (e2e/sc_kernels.py:333-354)."""
    return qkv_norm(epilogue(acc, xs, ws, 1), qn, kn, eps, L, hq, hk, d, **kw)


# ---------------------------------------------------------------------------------------------------------------
# a15-a18: MoE routing, grouped GEMM, combine.  e2e/sc_moe.py:114-185, e2e/fused_olmoe.py:34-66
# ---------------------------------------------------------------------------------------------------------------

def route_sort(inds, n_experts, tm):
    """Counting sort of the M*topk assignments by expert (e2e/sc_moe.py:114-155).  Order inside a segment is
    arbitrary in the reference (atomics); this restatement is the stable order, and `check_route` states the
    order-independent contract."""
    inds = np.asarray(inds, np.int64)
    M, k = inds.shape
    R = M * k
    flat = inds.reshape(-1)
    order = np.argsort(flat, kind="stable")
    pos = np.empty(R, np.int32)
    pos[order] = np.arange(R, dtype=np.int32)
    tok = np.zeros(R + tm, np.int32)
    tok[:R] = order // k
    esorted = flat[order].astype(np.int32)
    cnt = np.bincount(flat, minlength=n_experts)
    off = np.zeros(n_experts + 1, np.int32)
    off[1:] = np.cumsum(cnt)
    tstart = np.zeros(n_experts + 1, np.int32)
    tstart[1:] = np.cumsum(-(-cnt // tm))
    return pos, tok, esorted, off, tstart, -(-R // tm) + n_experts


def check_route(inds, n_experts, tm, pos, tok, esorted, off, tstart):
    """Order-independent contract of route_sort: pos is a permutation, every assignment lands inside its expert's
    segment, tok/esorted agree with pos, off/tstart are the prefix sums, padding rows gather token 0."""
    inds = np.asarray(inds, np.int64)
    M, k = inds.shape
    R = M * k
    flat = inds.reshape(-1)
    cnt = np.bincount(flat, minlength=n_experts)
    ok = np.array_equal(np.sort(pos), np.arange(R))
    ok &= np.array_equal(off, np.concatenate([[0], np.cumsum(cnt)]))
    ok &= np.array_equal(tstart, np.concatenate([[0], np.cumsum(-(-cnt // tm))]))
    ok &= bool(np.all((pos >= off[flat]) & (pos < off[flat + 1])))
    ok &= np.array_equal(tok[pos], np.arange(R) // k)
    ok &= np.array_equal(esorted[pos], flat)
    ok &= bool(np.all(tok[R:R + tm] == 0))
    return bool(ok)


def moe_mm(xq, R, wq_experts, off, epi, xs=None, ws_experts=None):
    """Grouped GEMM over expert segments (e2e/sc_moe.py:19-92; reference check :224-226): rows [off[e], off[e+1])
    use expert e's INT8 operand wq_experts[e] [N,K].  EPI 0 -> int32 [R,N]; EPI 1/3 -> bf16 values (float32)."""
    E = len(wq_experts)
    N = wq_experts[0].shape[0]
    acc = np.zeros((R, N), np.int32)
    wsr = np.zeros((R, N), np.float32)
    for e in range(E):
        a, b = int(off[e]), int(off[e + 1])
        if b > a:
            acc[a:b] = gemm_i32(xq[a:b], wq_experts[e])
            if ws_experts is not None:
                wsr[a:b] = ws_experts[e][None, :]
    if epi == 0:
        return acc
    a = (acc.astype(np.float32) * np.asarray(xs, np.float32)[:R, None]) * wsr
    y = bf16_round(a)
    if epi == 1:
        return y
    y4 = y.reshape(R, N // 4, 4)
    out = np.empty((R, N // 4, 2), np.float32)
    out[..., 0] = swiglu_bf16(y4[..., 0], y4[..., 2])
    out[..., 1] = swiglu_bf16(y4[..., 1], y4[..., 3])
    return out.reshape(R, N // 2)


def moe_combine(y, pos, scores, res, M):
    """h[t] = T(res[t] + acc_k), acc_j = rbf(rbf(y[pos[t*k+j]] * sc_j) + acc_{j-1}), j ascending; rows >= M copy
    res (e2e/fused_olmoe.py:45-66).  y, scores, res: float32 arrays holding bf16 values."""
    y = np.asarray(y, np.float32)
    res = np.asarray(res, np.float32)
    scores = np.asarray(scores, np.float32)
    k = scores.shape[1]
    h = res.copy()
    acc = np.zeros((M, res.shape[1]), np.float32)
    for j in range(k):
        p = np.asarray(pos).reshape(M, k)[:, j]
        acc = bf16_round(bf16_round(y[p] * scores[:M, j:j + 1]) + acc)
    h[:M] = bf16_round(res[:M] + acc)
    return h


def softmax_topk(logits, k):
    """Router: precise softmax over experts then the k largest, scores gathered without renormalisation
    (e2e/fused_olmoe.py:216-220 with norm_topk_prob False).  Order inside the top-k is by descending score with
    ties to the lower expert id; the reference's argpartition order is unspecified and only the SET matters for
    the expert GEMMs while the bf16 sum order follows the slot order it returns."""
    lg = np.asarray(logits, np.float32)
    m = lg.max(1, keepdims=True)
    p = np.exp((lg - m).astype(np.float32)).astype(np.float32)
    p = (p / p.sum(1, keepdims=True).astype(np.float32)).astype(np.float32)
    inds = np.argsort(-p, axis=1, kind="stable")[:, :k]
    return inds.astype(np.int32), np.take_along_axis(p, inds, 1)


# ---------------------------------------------------------------------------------------------------------------
# a19: decode GEMV, e2e/sc_decode.py:19-183
# ---------------------------------------------------------------------------------------------------------------

def gemv_i32(xq, wq):
    """tot[n] = sum_k xq[k] * q[n,k] as the exact integer (e2e/sc_decode.py:7-12,253)."""
    return (np.asarray(wq, np.int64) @ np.asarray(xq, np.int64)).astype(np.int32)


def gemv(xq, xs, wq, ws, epi, res=None):
    """Batch-1 W4A8 GEMV with the GEMM's epilogues (e2e/sc_decode.py:157-182).  Returns bf16 values as float32."""
    tot = gemv_i32(xq, wq)
    return epilogue(tot[None, :], np.asarray([xs], np.float32), ws, epi,
                    None if res is None else np.asarray(res, np.float32)[None, :])[0]
