"""Storage format of SC-MXFP4 weights and the GPU quantizer/packer.

Mirrors the interface of the reference's e2e/sc_format.py (Format, DEFAULT, pack_rows, decode_numpy,
from_shift_layout, quantize) so that callers written against it keep working:

  codes   uint32 [N * K / 8]   element k = 8 j + i of a row in bits 4 i .. 4 i + 3 of word j;  code = sign << 3 | idx
  bcodes  uint8  [N, K * bc_bits / (8 * block)]   block b of a row in bits bc_bits * (b % per_byte) of byte b // per_byte
  wscale  f32    [N]
  q[n, k] = +-code_mag[idx] * mult[bcode[n, k // block]],   W[n, k] = wscale[n] * q[n, k]

`quantize` runs on the GPU (scmx_quantize_sc_mxfp4, float64 arithmetic); the layout helpers are host-side NumPy.
"""
from dataclasses import dataclass

import numpy as np
import torch

from . import _lib


@dataclass(frozen=True)
class Format:
    """Same fields and checks as the reference's Format (e2e/sc_format.py:26-41)."""
    block: int = 32
    code_mag: tuple = (0, 1, 2, 3, 4, 6, 8, 12)
    mult: tuple = (1, 2, 4, 8)
    bc_bits: int = 2
    inline_mult: bool = False   # a Metal code-generation hint in the reference; accepted and ignored

    def __post_init__(self):
        assert self.block % 8 == 0, "a thread decodes 8 consecutive codes, which must share a block"
        assert self.bc_bits in (1, 2, 4, 8) and len(self.mult) <= 2 ** self.bc_bits
        assert len(self.code_mag) == 8 and max(self.code_mag) * max(self.mult) <= 127, "must fit INT8"

    @property
    def per_byte(self):
        return 8 // self.bc_bits

    def bits_per_weight(self, K):
        return 4 + self.bc_bits / self.block + 32 / K

    def c_struct(self):
        """The scmx_format passed down the C ABI."""
        assert len(self.mult) <= 16, "at most 16 block multipliers"
        f = _lib.ScmxFormat()
        f.block, f.bc_bits, f.n_mult = self.block, self.bc_bits, len(self.mult)
        for i, v in enumerate(self.code_mag):
            f.code_mag[i] = int(v)
        for i, v in enumerate(self.mult):
            f.mult[i] = int(v)
        return f


DEFAULT = Format()


def _or_fields(vals, bits):
    """Pack the last axis of small unsigned integers into one word, field i at bit offset bits * i."""
    shifts = (bits * np.arange(vals.shape[-1])).astype(vals.dtype)
    return np.bitwise_or.reduce(vals << shifts, axis=-1)


def pack_rows(code4, bcode, wscale, fmt=DEFAULT):
    """code4 uint8 [N, K] (sign << 3 | idx), bcode uint8 [N, K / block], wscale [N] -> (codes, bcodes, wscale)."""
    n, k = code4.shape
    assert k % fmt.block == 0
    nb = k // fmt.block
    assert nb % fmt.per_byte == 0 and bcode.max() < len(fmt.mult)
    codes = _or_fields(code4.astype(np.uint32).reshape(n, k // 8, 8), 4).astype(np.uint32)
    bc = _or_fields(bcode.astype(np.uint32).reshape(n, nb // fmt.per_byte, fmt.per_byte), fmt.bc_bits).astype(np.uint8)
    return codes.reshape(-1), bc, np.asarray(wscale, np.float32)


def decode_numpy(codes, bc, n, k, fmt=DEFAULT):
    """Host-side decode of the packed layout to the INT8 operand q [N, K]."""
    words = np.asarray(codes, np.uint32).reshape(n, k // 8, 1)
    c = ((words >> (4 * np.arange(8, dtype=np.uint32))) & 0xF).reshape(n, k).astype(np.int32)
    bytes_ = np.asarray(bc, np.uint8).reshape(n, -1, 1).astype(np.uint32)
    b = ((bytes_ >> (fmt.bc_bits * np.arange(fmt.per_byte, dtype=np.uint32))) & (2 ** fmt.bc_bits - 1))
    b = b.reshape(n, k // fmt.block).astype(np.int32)
    mag = np.asarray(fmt.code_mag)[c & 7] * np.repeat(np.asarray(fmt.mult)[b], fmt.block, axis=1)
    return np.where(c & 8, -mag, mag).astype(np.int8)


def from_shift_layout(codes_u32, shifts, wscale, fmt=DEFAULT):
    """Byte-shift layout (codes uint32 [N*K/8], shifts uint8 [N, K/32] in 0..3, wscale [N]) -> this format's packed
    block codes, without requantizing."""
    assert fmt.block == 32 and tuple(fmt.mult) == (1, 2, 4, 8), "shift layout is the power-of-two BLOCK=32 format"
    n, nb = shifts.shape
    bc = _or_fields(np.asarray(shifts, np.uint32).reshape(n, nb // fmt.per_byte, fmt.per_byte), fmt.bc_bits)
    return np.asarray(codes_u32, np.uint32).reshape(-1), bc.astype(np.uint8), np.asarray(wscale, np.float32)


def pack_values(v, e, fmt=DEFAULT):
    """Packing from E2M1 values v [N, K/32, 32] (levels 0, 0.5, 1, 1.5, 2, 3, 4, 6 with sign) and block exponents
    e [N, K/32] instead of from weights - for roundings other than round-to-nearest that keep the exponents of the
    unquantized weights, as the reference's GPTQ pack does (pack_ve, e2e/gptq_pack.py:29-47).  Host-side NumPy like the
    other layout helpers.  Returns (codes uint32 [N*K/8], bcodes uint8 [N, K/128], wscale f32 [N], qw int8 [N, K]).
    A non-finite exponent marks an all-zero block."""
    assert fmt.block == 32 and tuple(fmt.mult) == (1, 2, 4, 8) and fmt.bc_bits == 2
    v = np.asarray(v, np.float64)
    e = np.asarray(e, np.float64)
    n, nb, blk = v.shape
    assert blk == 32 and e.shape == (n, nb) and nb % fmt.per_byte == 0
    fin = np.isfinite(e)
    hi = np.where(fin, e, -np.inf).max(-1, keepdims=True)
    hi = np.where(np.isfinite(hi), hi, 0.0)
    lo = np.where(fin, e, hi).min(-1, keepdims=True)
    spread = np.where(fin, e, lo) - lo
    if spread.max() > 3:
        raise ValueError(f"block exponent spread {int(spread.max())} > 3: not INT8-embeddable")
    levels = np.asarray(fmt.code_mag, np.float64) / 2
    a = np.abs(v)
    idx = np.searchsorted(levels, a)
    if idx.max() > 7 or not np.array_equal(levels[np.minimum(idx, 7)], a):
        raise ValueError("values are not E2M1 levels")
    if np.any(a[~fin] != 0):
        raise ValueError("a block without an exponent holds non-zero values")
    code4 = (idx | ((v < 0) << 3)).astype(np.uint8).reshape(n, nb * 32)
    shifts = spread.astype(np.uint8)
    codes, bc, ws = pack_rows(code4, shifts, np.exp2(lo[:, 0] - 1).astype(np.float32), fmt)
    return codes, bc, ws, decode_numpy(codes, bc, n, nb * 32, fmt).astype(np.int8)


_DTYPE_CODE = {torch.float32: 0, torch.float64: 1, torch.bfloat16: 2}


def quantize_device(w, fmt=DEFAULT, want_qw=True):
    """SC-MXFP4 quantize + pack of a CUDA tensor w [N, K] (float32 / float64 / bfloat16) on the GPU.
    Returns CUDA tensors (codes int32-viewed-uint32 [N*K/8], bcodes uint8 [N, K/128], wscale f32 [N], qw int8 [N, K]
    or None, row_exp int32 [N])."""
    assert fmt.block == 32 and tuple(fmt.mult) == (1, 2, 4, 8) and fmt.bc_bits == 2, "SC-MXFP4 is BLOCK=32, MULT=2^shift"
    assert tuple(fmt.code_mag) == DEFAULT.code_mag
    _lib.require_cuda(w)
    assert w.dim() == 2 and w.dtype in _DTYPE_CODE, "w must be a 2-D float32/float64/bfloat16 CUDA tensor"
    n, k = w.shape
    assert k % 128 == 0, f"K={k} must be a multiple of 128"
    dev = w.device
    codes = torch.empty(n * k // 8, dtype=torch.int32, device=dev)
    bcodes = torch.empty((n, k // 128), dtype=torch.uint8, device=dev)
    wscale = torch.empty(n, dtype=torch.float32, device=dev)
    qw = torch.empty((n, k), dtype=torch.int8, device=dev) if want_qw else None
    row_exp = torch.empty(n, dtype=torch.int32, device=dev)
    with torch.cuda.device(dev):
        _lib.call("scmx_quantize_sc_mxfp4", _lib.ptr(w), _DTYPE_CODE[w.dtype], n, k, _lib.ptr(codes), _lib.ptr(bcodes),
                  _lib.ptr(wscale), _lib.ptr(qw), _lib.ptr(row_exp), _lib.stream())
    return codes, bcodes, wscale, qw, row_exp


def quantize(w, fmt=DEFAULT):
    """(N, K) float weights -> (codes, bcodes, wscale, qw).  NumPy in -> NumPy out (uint32 / uint8 / f32 / int8), like the
    reference; a CUDA tensor in -> CUDA tensors out.  The arithmetic always runs on the GPU in float64."""
    if isinstance(w, torch.Tensor):
        c, b, s, q, _ = quantize_device(w.contiguous(), fmt)
        return c, b, s, q
    wt = torch.from_numpy(np.ascontiguousarray(np.asarray(w, dtype=np.float64))).cuda()
    c, b, s, q, _ = quantize_device(wt, fmt)
    return (c.cpu().numpy().view(np.uint32), b.cpu().numpy(), s.cpu().numpy(), q.cpu().numpy())


def family_quantize_device(w, fmt, base_grid=8):
    """Integer-exact family quantizer (row base x block multiplier search, float32) on the GPU for a generic Format.
    Returns CUDA tensors (codes, bcodes, wscale = row base, qw)."""
    _lib.require_cuda(w)
    assert w.dim() == 2 and w.dtype == torch.float32
    n, k = w.shape
    nb = k // fmt.block
    assert k % fmt.block == 0 and nb % fmt.per_byte == 0 and nb % 8 == 0 and 8 <= nb <= 128, \
        "rows must have between 8 and 128 blocks, a multiple of 8"
    dev = w.device
    codes = torch.empty(n * k // 8, dtype=torch.int32, device=dev)
    bcodes = torch.empty((n, nb // fmt.per_byte), dtype=torch.uint8, device=dev)
    wscale = torch.empty(n, dtype=torch.float32, device=dev)
    qw = torch.empty((n, k), dtype=torch.int8, device=dev)
    f = fmt.c_struct()
    with torch.cuda.device(dev):
        _lib.call("scmx_quantize_family", _lib.ptr(w), n, k, f, base_grid, _lib.ptr(codes), _lib.ptr(bcodes),
                  _lib.ptr(wscale), _lib.ptr(qw), _lib.stream())
    return codes, bcodes, wscale, qw


def to_device(codes, bcodes, wscale, device="cuda"):
    """NumPy packed arrays -> CUDA tensors in the dtypes the kernels take (codes reinterpreted as int32)."""
    c = torch.from_numpy(np.ascontiguousarray(np.asarray(codes, np.uint32)).view(np.int32)).to(device)
    b = torch.from_numpy(np.ascontiguousarray(np.asarray(bcodes, np.uint8))).to(device)
    s = torch.from_numpy(np.ascontiguousarray(np.asarray(wscale, np.float32))).to(device)
    return c, b, s
