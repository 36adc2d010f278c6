"""Prefill-side kernels of the W4A8 path as torch functions, with the call signatures of the reference's
e2e/sc_kernels.py: every function takes M rows and writes Mp >= M rows (rows >= M are zero), returns freshly
allocated CUDA tensors, and accepts (and ignores) the reference's Metal tuning arguments `deps`, `tile`, `nt`.

  act_quant, unpack_i8, mm_i8_i32, mm_epi, rmsnorm_quant, rmsnorm_quant_n, res_norm_quant, res_epilogue,
  swiglu_quant, interleave_gate_up, pad_rows, set_format

All arithmetic happens in libscmx (CUDA, sm_100a); the GEMMs are tcgen05 kind::i8 kernels.
"""
import numpy as np
import torch

from . import _lib
from . import sc_format as F

TM, TN, NSG, GROUP_M = 128, 256, 4, 8   # M tile of the GEMM kernel (row padding unit); the rest are informational


def set_format(fmt):
    """Switch every kernel (unpack, grouped expert GEMM, GEMV) to another weight format (sc_format.Format)."""
    F.DEFAULT = fmt


def pad_rows(M):
    return -(-M // TM) * TM


def _bf16(x):
    assert x.dtype == torch.bfloat16, "activations are bfloat16"
    return x


def unpack_i8(codes, bcodes, N, K, deps=(), out=None):
    """Packed codes + block codes -> INT8 operand [N, K] (written into `out` when given)."""
    _lib.require_cuda(codes, bcodes, out)
    wq = out if out is not None else torch.empty((N, K), dtype=torch.int8, device=codes.device)
    assert wq.dtype == torch.int8 and wq.numel() >= N * K
    _lib.call("scmx_unpack_i8", _lib.ptr(codes), _lib.ptr(bcodes), N, K, F.DEFAULT.c_struct(), _lib.ptr(wq), _lib.stream())
    return wq


def act_quant(x, Mp=None, nt=256, deps=()):
    """x bf16 [M, K] -> (xq int8 [Mp, K], xscale f32 [Mp]): per-token symmetric INT8, rows >= M zero."""
    _lib.require_cuda(x)
    M, K = _bf16(x).shape
    Mp = Mp or pad_rows(M)
    xq = torch.empty((Mp, K), dtype=torch.int8, device=x.device)
    xs = torch.empty(Mp, dtype=torch.float32, device=x.device)
    _lib.call("scmx_act_quant", _lib.ptr(x), M, K, Mp, _lib.ptr(xq), _lib.ptr(xs), _lib.stream())
    return xq, xs


def act_quant_seg(xseg, Mp=None):
    """act_quant of rows stored as column segments: xseg bf16 [G, M, w] holds the [M, G*w] matrix whose columns
    g*w .. (g+1)*w are xseg[g] (what an all-gather of column shards produces)."""
    _lib.require_cuda(xseg)
    G, M, w = _bf16(xseg).shape
    Mp = Mp or pad_rows(M)
    xq = torch.empty((Mp, G * w), dtype=torch.int8, device=xseg.device)
    xs = torch.empty(Mp, dtype=torch.float32, device=xseg.device)
    _lib.call("scmx_act_quant_seg", _lib.ptr(xseg), M, G * w, Mp, G, M * w, _lib.ptr(xq), _lib.ptr(xs), _lib.stream())
    return xq, xs


def rmsnorm_quant_seg(xseg, w, eps, Mp=None):
    """rmsnorm_quant of rows stored as column segments (see act_quant_seg)."""
    _lib.require_cuda(xseg, w)
    G, M, ws = _bf16(xseg).shape
    Mp = Mp or pad_rows(M)
    xq = torch.empty((Mp, G * ws), dtype=torch.int8, device=xseg.device)
    xs = torch.empty(Mp, dtype=torch.float32, device=xseg.device)
    _lib.call("scmx_rmsnorm_quant_seg", _lib.ptr(xseg), _lib.ptr(w), _eps(eps), M, G * ws, Mp, G, M * ws, _lib.ptr(xq),
              _lib.ptr(xs), None, _lib.stream())
    return xq, xs


def _eps(eps):
    return float(eps.reshape(-1)[0].item()) if isinstance(eps, torch.Tensor) else float(eps)


def rmsnorm_quant(x, w, eps, Mp=None, deps=()):
    """x [M, K] -> (xq int8 [Mp, K], xscale f32 [Mp]) of rms_norm(x, w, eps)."""
    xq, xs, _ = _rmsnorm_quant(x, w, eps, Mp, False)
    return xq, xs


def rmsnorm_quant_n(x, w, eps, Mp=None, deps=()):
    """rmsnorm_quant that also returns the normalized bf16 rows: (xq, xscale, xn [Mp, K])."""
    return _rmsnorm_quant(x, w, eps, Mp, True)


def _rmsnorm_quant(x, w, eps, Mp, want_n):
    _lib.require_cuda(x, w)
    M, K = _bf16(x).shape
    assert w.shape == (K,) and w.dtype == torch.bfloat16
    Mp = Mp or pad_rows(M)
    xq = torch.empty((Mp, K), dtype=torch.int8, device=x.device)
    xs = torch.empty(Mp, dtype=torch.float32, device=x.device)
    xn = torch.empty((Mp, K), dtype=torch.bfloat16, device=x.device) if want_n else None
    _lib.call("scmx_rmsnorm_quant", _lib.ptr(x), _lib.ptr(w), _eps(eps), M, K, Mp, _lib.ptr(xq), _lib.ptr(xs),
              _lib.ptr(xn), _lib.stream())
    return xq, xs, xn


def mm_i8_i32(xq, wq, deps=(), tile=None):
    """INT8 [M, K] x INT8 [N, K]^T -> INT32 [M, N] (exact)."""
    _lib.require_cuda(xq, wq)
    (M, K), N = xq.shape, wq.shape[0]
    assert xq.dtype == torch.int8 and wq.dtype == torch.int8 and wq.shape[1] == K
    assert M % TM == 0 and N % 32 == 0, (M, N, TM)
    acc = torch.empty((M, N), dtype=torch.int32, device=xq.device)
    _lib.call("scmx_mm_i8", _lib.ptr(xq), _lib.ptr(wq), M, N, K, 0, None, None, None, _lib.ptr(acc),
              _lib.ptr(_lib.status_buffer()), _lib.stream())
    return acc


def mm_epi(xq, wq, xscale, wscale, epi, dtype=torch.bfloat16, res=None, deps=(), tile=None):
    """INT8 GEMM + fused epilogue (EPI 1: scaled bf16, 2: + residual, 3: SwiGLU of interleaved gate/up -> [M, N/2])."""
    _lib.require_cuda(xq, wq, xscale, wscale, res)
    (M, K), N = xq.shape, wq.shape[0]
    assert dtype == torch.bfloat16, "outputs are bfloat16"
    assert epi in (1, 2, 3)
    assert M % TM == 0 and N % 32 == 0 and (epi != 2 or tuple(res.shape) == (M, N)), (M, N, TM)
    assert xscale.shape == (M,) and wscale.shape == (N,)
    out = torch.empty((M, N // 2 if epi == 3 else N), dtype=torch.bfloat16, device=xq.device)
    _lib.call("scmx_mm_i8", _lib.ptr(xq), _lib.ptr(wq), M, N, K, epi, _lib.ptr(xscale), _lib.ptr(wscale),
              _lib.ptr(res) if epi == 2 else None, _lib.ptr(out), _lib.ptr(_lib.status_buffer()), _lib.stream())
    return out


def mm_w4_epi(xq, codes, bcodes, xscale, wscale, N, epi, dtype=torch.bfloat16, res=None):
    """mm_epi(xq, unpack_i8(codes, bcodes, N, K), ...) as ONE kernel: the packed weight tiles are expanded to INT8 in shared
    memory inside the K loop (the single-pass form of the reference, kernels/w4a8.metal:78-155), so no INT8 copy of the
    weights is written.  Same bits as the two-kernel form.  epi 0 returns the INT32 accumulators."""
    _lib.require_cuda(xq, codes, bcodes, xscale, wscale, res)
    M, K = xq.shape
    assert dtype == torch.bfloat16 and epi in (0, 1, 2, 3)
    assert M % TM == 0 and N % 32 == 0 and (epi != 2 or tuple(res.shape) == (M, N))
    fmt = F.DEFAULT
    assert _lib.lib().scmx_w4_supported(fmt.c_struct(), K), "format / K not covered by the packed-weight GEMM"
    out = torch.empty((M, N), dtype=torch.int32, device=xq.device) if epi == 0 else \
        torch.empty((M, N // 2 if epi == 3 else N), dtype=torch.bfloat16, device=xq.device)
    _lib.call("scmx_mm_w4", _lib.ptr(xq), _lib.ptr(codes), _lib.ptr(bcodes), M, N, K, fmt.c_struct(), epi, _lib.ptr(xscale),
              _lib.ptr(wscale), _lib.ptr(res) if epi == 2 else None, _lib.ptr(out), _lib.ptr(_lib.status_buffer()), _lib.stream())
    return out


def interleave_gate_up(Fdim):
    """Row permutation of [gate (F rows); up (F rows)] into groups g_2p, g_2p+1, u_2p, u_2p+1 for EPI 3."""
    p = np.arange(Fdim // 2)
    return np.stack([2 * p, 2 * p + 1, Fdim + 2 * p, Fdim + 2 * p + 1], 1).reshape(-1)


def res_epilogue(acc, xscale, wscale, res, deps=()):
    """h = res + bf16(acc * xscale * wscale) from INT32 accumulators."""
    _lib.require_cuda(acc, xscale, wscale, res)
    Mp, N = acc.shape
    assert res.shape == (Mp, N) and res.dtype == torch.bfloat16 and acc.dtype == torch.int32
    h = torch.empty((Mp, N), dtype=torch.bfloat16, device=acc.device)
    _lib.call("scmx_res_epilogue", _lib.ptr(acc), _lib.ptr(xscale), _lib.ptr(wscale), _lib.ptr(res), Mp, N, _lib.ptr(h),
              _lib.stream())
    return h


def res_norm_quant(acc, xscale, wscale, res, w, eps, deps=()):
    """h = res + bf16(acc * xscale * wscale); returns (h [Mp, K], xq, xscale') of rms_norm(h)."""
    h = res_epilogue(acc, xscale, wscale, res)
    xq, xs = rmsnorm_quant(h, w, eps, h.shape[0])
    return h, xq, xs


def swiglu_quant(acc, xscale, wscale, dtype=torch.bfloat16, nt=512, deps=()):
    """acc int32 [Mp, 2F] (gate | up) -> (xq int8 [Mp, F], xscale f32 [Mp]) of swiglu(bf16 gate, bf16 up)."""
    _lib.require_cuda(acc, xscale, wscale)
    Mp, F2 = acc.shape
    Fd = F2 // 2
    assert acc.dtype == torch.int32 and Fd % 4 == 0
    xq = torch.empty((Mp, Fd), dtype=torch.int8, device=acc.device)
    xs = torch.empty(Mp, dtype=torch.float32, device=acc.device)
    _lib.call("scmx_swiglu_quant", _lib.ptr(acc), _lib.ptr(xscale), _lib.ptr(wscale), Mp, Fd, _lib.ptr(xq), _lib.ptr(xs),
              _lib.stream())
    return xq, xs


def sc_swiglu(g, u):
    """Elementwise bf16-stepwise SiLU(g) * u (the device function of the EPI 3 epilogue) on bf16 tensors."""
    _lib.require_cuda(g, u)
    assert g.dtype == torch.bfloat16 and u.dtype == torch.bfloat16 and g.shape == u.shape
    out = torch.empty_like(g)
    _lib.call("scmx_swiglu", _lib.ptr(g), _lib.ptr(u), g.numel(), _lib.ptr(out), _lib.stream())
    return out


def rot_signs(K, device="cuda"):
    """The +-1 sign vector for input width K: numpy.random.default_rng(0).choice([-1, 1], K), one per width so that q/k/v
    and gate/up share a rotated input (e2e/sc_kernels.py:566-569)."""
    return torch.from_numpy(np.random.default_rng(0).choice([-1.0, 1.0], size=K).astype(np.float32)).to(device)


def rot_quant(x, signs, Mp=None, nt=512, deps=()):
    """x bf16 [M, K] -> (xq int8 [Mp, K], xscale f32 [Mp]): sign flip and 32-point Hadamard rotation of each 32-wide block,
    then per-token INT8."""
    _lib.require_cuda(x, signs)
    M, K = _bf16(x).shape
    assert signs.shape == (K,) and signs.dtype == torch.float32
    Mp = Mp or pad_rows(M)
    xq = torch.empty((Mp, K), dtype=torch.int8, device=x.device)
    xs = torch.empty(Mp, dtype=torch.float32, device=x.device)
    _lib.call("scmx_rot_quant", _lib.ptr(x), _lib.ptr(signs), M, K, Mp, _lib.ptr(xq), _lib.ptr(xs), _lib.stream())
    return xq, xs


def rope_inv_freq(d, base, device="cuda"):
    """f32 [d/2]: base^(-2i/d), the frequencies of a half-split (non-interleaved) rotary embedding."""
    i = torch.arange(0, d, 2, dtype=torch.float64, device=device)   # device=None: torch's current default device
    return (1.0 / (float(base) ** (i / d))).to(torch.float32)


def rope_table(inv_freq, rows):
    """f32 [rows, d]: cos then sin of position * inv_freq (the product in float32, the functions in float64, rounded to
    float32): what the q/k/v kernel evaluates per call, precomputed."""
    ang = (torch.arange(rows, device=inv_freq.device, dtype=torch.float32)[:, None] * inv_freq[None, :]).double()
    return torch.cat([torch.cos(ang), torch.sin(ang)], 1).float().contiguous()


def _qkv_norm(src, xscale, wscale, qn, kn, eps, L, hq, hk, d, full, rope, cache, pos_dev=None):
    _lib.require_cuda(src, xscale, wscale, qn, kn)
    ntot = (hq + 2 * hk) * d
    assert src.shape[1] == ntot and src.shape[0] >= L and src.is_contiguous()
    is_acc = src.dtype == torch.int32
    assert is_acc or src.dtype == torch.bfloat16
    inv_freq, pos0 = (rope[0], rope[1]) if rope is not None else (None, 0)
    table = rope[2] if rope is not None and len(rope) > 2 else None      # optional rope_table(...) of the same inv_freq
    q = torch.empty((hq, L, d), dtype=torch.bfloat16, device=src.device)
    if cache is None:
        k = torch.empty((hk, L, d), dtype=torch.bfloat16, device=src.device)
        v = torch.empty_like(k)
        kbuf, vbuf, cap, row0 = k, v, L, 0
    else:
        kbuf, vbuf, cap, row0 = cache.k, cache.v, cache.k.shape[1], cache.offset
        assert kbuf.shape == (hk, cap, d) and kbuf.is_contiguous() and vbuf.is_contiguous()
        k, v = kbuf[:, :row0 + L], vbuf[:, :row0 + L]
    _lib.call("scmx_qkv_norm", _lib.ptr(src), int(is_acc), _lib.ptr(xscale), _lib.ptr(wscale), _lib.ptr(qn), _lib.ptr(kn),
              _eps(eps), L, hq, hk, d, int(full), _lib.ptr(inv_freq), _lib.ptr(table),
              0 if table is None else table.shape[0], int(pos0), _lib.ptr(pos_dev), _lib.ptr(q), L,
              _lib.ptr(kbuf), _lib.ptr(vbuf), cap, row0, _lib.stream())
    return q, k, v


def qkv_epilogue_headnorm(acc, xscale, wscale, qn, kn, eps, L, hq, hk, d, dtype=torch.bfloat16, deps=(), rope=None,
                          cache=None):
    """acc int32 [Mp, (hq + 2 hk) d] -> q [hq, L, d], k [hk, L, d], v [hk, L, d] with per-head RMSNorm of q and k.
    rope=(inv_freq, pos0[, rope_table]): rotary embedding of q and k at positions pos0.. in the same kernel; cache (with .k, .v
    [hk, capacity, d] and .offset): k and v are written into the cache rows and the filled prefix is returned."""
    return _qkv_norm(acc, xscale, wscale, qn, kn, eps, L, hq, hk, d, False, rope, cache)


def qkv_headnorm_y(y, qn, kn, eps, L, hq, hk, d, deps=(), rope=None, cache=None, pos_dev=None):
    """bf16 y [Mp, (hq + 2 hk) d] -> q [hq, L, d], k [hk, L, d], v [hk, L, d] (q/k per-head RMSNorm)."""
    return _qkv_norm(y, None, None, qn, kn, eps, L, hq, hk, d, False, rope, cache, pos_dev)


def qkv_fullnorm_y(y, qn, kn, eps, L, h, d, deps=(), rope=None, cache=None, pos_dev=None):
    """bf16 y [Mp, 3 h d] -> q, k, v [h, L, d] with RMSNorm over the full h*d-wide q and k."""
    return _qkv_norm(y, None, None, qn, kn, eps, L, h, h, d, True, rope, cache, pos_dev)


class DecodeAttention:
    """Batch-1 attention over a KV cache (scmx_attn_decode) with its scratch: q [hq, 1, d] or [hq, d], cache with .k / .v
    [hk, capacity, d] -> bf16 [1, hq * d].  n_pos positions are attended, or pos_dev[0] + 1 when pos_dev (int32 [1] on the
    device) is given, which keeps the call replayable from a CUDA graph while the sequence grows."""

    def __init__(self, hq, hk, d, device="cuda", n_sm=148):
        self.hq, self.hk, self.d = hq, hk, d
        self.nsplit = max(1, min(32, n_sm // hk))
        self.part = torch.empty((hq, self.nsplit, d + 2), dtype=torch.float32, device=device)
        self.counters = torch.zeros(hk, dtype=torch.int32, device=device)

    @staticmethod
    def supports(hq, hk, d):
        return d in (64, 128) and hq % hk == 0 and hq // hk in (1, 2, 4)

    def __call__(self, q, cache, scale, n_pos=None, pos_dev=None):
        _lib.require_cuda(q, cache.k, cache.v, pos_dev)
        assert q.dtype == torch.bfloat16 and q.is_contiguous() and q.numel() == self.hq * self.d
        out = torch.empty((1, self.hq * self.d), dtype=torch.bfloat16, device=q.device)
        _lib.call("scmx_attn_decode", _lib.ptr(q), _lib.ptr(cache.k), _lib.ptr(cache.v), cache.k.shape[1], _lib.ptr(pos_dev),
                  int(n_pos or 0), float(scale), self.hq, self.hk, self.d, self.nsplit, _lib.ptr(self.part),
                  _lib.ptr(self.counters), _lib.ptr(out), _lib.stream())
        return out


def set_gemm_tile(bn=0):
    """Tuning hint for the GEMM N tile (0 automatic, 128, 256)."""
    _lib.call("scmx_set_gemm_tile", bn)
