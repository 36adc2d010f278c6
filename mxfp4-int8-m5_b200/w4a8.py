"""Unfused W4A8 linear layer and weight packing, mirroring the reference's e2e/w4a8_mlx.py (W4A8Linear, pack_linear)
and the row-concatenated PackedWeight of e2e/fused_qwen3.py:35-59, as torch modules over libscmx."""
import numpy as np
import torch

from . import sc_format as F
from . import sc_kernels as S


def pack_linear(w):
    """(N, K) float weights -> (codes uint32 [N*K/8], shifts uint8 [N, K/32], wscale f32 [N]) as NumPy: the byte-shift
    layout of the reference's pack_linear (one shift byte per 32-block)."""
    codes, bc, ws, _ = F.quantize(np.asarray(w, dtype=np.float64))
    shifts = ((bc[..., None] >> (2 * np.arange(4, dtype=np.uint8))) & 3).reshape(bc.shape[0], -1).astype(np.uint8)
    return codes, shifts, ws


class PackedWeight:
    """Row concatenation of packed matrices (exact: the format is per output row), optional row permutation
    (e.g. interleave_gate_up for the SwiGLU epilogue); holds CUDA tensors."""

    def __init__(self, parts, perm=None, resident=False, device="cuda"):
        """parts: list of (codes [N*K/8], bcodes [N, K/128], wscale [N]) as NumPy arrays (uint32 / uint8 / f32) or as the
        CUDA tensors quantize_device returns."""
        dev = device

        def cu(x, np_dtype):
            if isinstance(x, torch.Tensor):
                return x.to(dev)
            a = np.ascontiguousarray(np.asarray(x, np_dtype))
            return torch.from_numpy(a.view(np.int32) if np_dtype == np.uint32 else a).to(dev)

        self.splits = [int(p[2].shape[0]) for p in parts]
        codes = torch.cat([cu(p[0], np.uint32).reshape(n, -1) for p, n in zip(parts, self.splits)])
        bc = torch.cat([cu(p[1], np.uint8) for p in parts])
        ws = torch.cat([cu(p[2], np.float32) for p in parts])
        self.perm = perm
        if perm is not None:
            idx = torch.as_tensor(np.asarray(perm), device=dev, dtype=torch.long)
            codes, bc, ws = codes[idx], bc[idx], ws[idx]
        self.N, self.K = codes.shape[0], codes.shape[1] * 8
        self.codes, self.bcodes, self.wscale = codes.reshape(-1).contiguous(), bc.contiguous(), ws.contiguous()
        self.wq = S.unpack_i8(self.codes, self.bcodes, self.N, self.K) if resident else None

    def int8(self):
        return self.wq if self.wq is not None else S.unpack_i8(self.codes, self.bcodes, self.N, self.K)

    def unpack(self, deps=()):
        return self.int8()

    def nbytes(self):
        return self.codes.numel() * 4 + self.bcodes.numel() + self.wscale.numel() * 4

    def entry(self):
        """(codes, bcodes, wscale, N, K) as the chained calls take it."""
        return self.codes, self.bcodes, self.wscale, self.N, self.K


class W4A8Linear(torch.nn.Module):
    """Bias-free linear y = x W^T with SC-MXFP4 weights computed as INT8 x INT8 on the tensor cores:
    act_quant -> (unpack) -> tcgen05 GEMM with the scaling epilogue.  resident_int8=True keeps the unpacked INT8
    operand in memory instead of decoding it per call."""

    def __init__(self, codes, shifts, wscale, resident_int8=False, device="cuda"):
        super().__init__()
        shifts = np.asarray(shifts, np.uint8)
        self.N = shifts.shape[0]
        self.K = np.asarray(codes).size * 8 // self.N
        if shifts.shape[1] * 32 == self.K:                 # one shift byte per 32-block (the reference's pack_linear)
            c, b, s = F.from_shift_layout(np.asarray(codes, np.uint32), shifts, wscale)
        else:                                              # already 2-bit block codes, four blocks per byte
            c, b, s = np.asarray(codes, np.uint32), shifts, wscale
        self.codes, self.bcodes, self.wscale = F.to_device(c, b, s, device)
        self.wq = S.unpack_i8(self.codes, self.bcodes, self.N, self.K) if resident_int8 else None

    def int8_weight(self):
        return self.wq if self.wq is not None else S.unpack_i8(self.codes, self.bcodes, self.N, self.K)

    def forward(self, x):
        lead, K = x.shape[:-1], x.shape[-1]
        x2 = x.reshape(-1, K).to(torch.bfloat16).contiguous()
        M = x2.shape[0]
        xq, xs = S.act_quant(x2)                      # pads to a multiple of the M tile; padded rows are zero
        y = S.mm_epi(xq, self.int8_weight(), xs, self.wscale, 1)
        return y[:M].reshape(*lead, self.N).to(x.dtype)


def apply_w4a8(model, packed, resident_int8=False):
    """Swaps every transformer-block linear of a host_model.CausalLM for W4A8Linear (embeddings, norms, attention and the
    output head unchanged), e2e/w4a8_mlx.py:197-207.  packed: {"layers.{i}.{path}": (codes, shifts or bcodes, wscale)}."""
    from .host_model import LINEARS
    dev = model.model.embed_tokens.weight.device
    for i, layer in enumerate(model.model.layers):
        for path in LINEARS:
            parent_name, name = path.split(".")
            parent = getattr(layer, parent_name)
            setattr(parent, name, W4A8Linear(*packed[f"layers.{i}.{path}"], resident_int8=resident_int8, device=dev))
    return model
