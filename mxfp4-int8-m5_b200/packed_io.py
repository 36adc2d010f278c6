"""On-disk interchange of packed SC-MXFP4 weights: one safetensors file with the reference's key scheme, and the view that
lets MXFP4 kernels read the same code words.

  layers.{i}.{path}.codes | .bcodes | .wscale        e2e/pack_format.py:101-108, e2e/fused_olmoe.py:117-125
  layers.{i}.{path}.codes | .shifts | .wscale        the byte-shift cache of e2e/w4a8_mlx.py:176-196
  layers.{i}.experts.{gate_proj|up_proj|down_proj}.{e}.codes | ...

Arrays are NumPy on the host side of the file (codes uint32, bcodes / shifts uint8, wscale float32); files written by the
reference load unchanged and the other way round.
"""
import os

import numpy as np
from safetensors.numpy import load_file, save_file

from . import sc_format as F

SUFFIXES = (".codes", ".bcodes", ".wscale")


def save_packed(path, packed):
    """packed: {name: (codes, bcodes, wscale)} -> one safetensors file, written under a temporary name first."""
    flat = {}
    for name, (c, b, s) in packed.items():
        c = np.asarray(c)
        flat[name + ".codes"] = np.ascontiguousarray((c.view(np.uint32) if c.dtype == np.int32 else c.astype(np.uint32)).reshape(-1))
        flat[name + ".bcodes"] = np.ascontiguousarray(np.asarray(b, np.uint8))
        flat[name + ".wscale"] = np.ascontiguousarray(np.asarray(s, np.float32))
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    tmp = path + ".tmp"
    save_file(flat, tmp)
    os.replace(tmp, path)


def load_packed(path, fmt=F.DEFAULT):
    """-> {name: (codes, bcodes, wscale)}; entries stored with one shift byte per 32-block (".shifts") are converted to
    2-bit block codes (e2e/fused_qwen3.py:62-73)."""
    flat = load_file(path)
    out = {}
    for key in flat:
        if not key.endswith(".codes"):
            continue
        name = key[:-len(".codes")]
        if name + ".bcodes" in flat:
            out[name] = (flat[key], flat[name + ".bcodes"], flat[name + ".wscale"])
        else:
            out[name] = F.from_shift_layout(flat[key], flat[name + ".shifts"], flat[name + ".wscale"], fmt)
    return out


def mxfp4_scales(bcodes, wscale, K, fmt=F.DEFAULT):
    """uint8 E8M0 scales [N, K / 32] under which an MXFP4 decoder (value = e2m1(nibble) * 2^(scale - 127)) reads the
    packed code words as the same weights: the nibble is sign << 3 | index into 2 x E2M1 magnitudes, so
    w = wscale * 2 * e2m1 * 2^shift and scale = log2(wscale) + 1 + shift + 127 (e2e/fused_qwen38.py:319-334).
    Only for the SC-MXFP4 format itself: blocks of 32, shifts, power-of-two row scales."""
    assert fmt.block == 32 and tuple(fmt.mult) == (1, 2, 4, 8) and tuple(fmt.code_mag) == (0, 1, 2, 3, 4, 6, 8, 12)
    bc = np.asarray(bcodes, np.uint8)
    b = np.arange(K // 32)
    shifts = (bc[:, b // fmt.per_byte] >> (fmt.bc_bits * (b % fmt.per_byte)).astype(np.uint8)) & ((1 << fmt.bc_bits) - 1)
    mant, exp = np.frexp(np.asarray(wscale, np.float64))          # wscale = mant * 2^exp, mant = 0.5 for powers of two
    if not np.all(mant == 0.5):
        raise ValueError("row scale is not a power of two")
    e = (exp - 1)[:, None] + 1 + shifts.astype(np.int64) + 127
    if e.min() < 0 or e.max() > 254:
        raise ValueError("scale outside the E8M0 range")
    return np.ascontiguousarray(e.astype(np.uint8))
