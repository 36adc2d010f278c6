"""Fused SC-MXFP4 W4A8 prefill for Qwen3-style dense decoders: the torch counterpart of the reference's FusedQwen3
(e2e/fused_qwen3.py:82-301) over libscmx.  Per block:

    [xq, xs = rmsnorm_quant(h)]                      (input RMSNorm + INT8; the previous block ends with it)
    y = mm_epi(xq, unpack(Wq|Wk|Wv), EPI 1)          one GEMM on the row-concatenated projections
    q, k, v = qkv_headnorm_y(y)                      per-head q/k RMSNorm + rotary embedding + KV-cache append, one kernel
    o = sdpa(q, k, v)                                torch's attention, outside the W4A8 path
    h = mm_epi(act_quant(o), unpack(Wo), EPI 2, res=h)
    act = mm_epi(rmsnorm_quant(h), unpack(Wg|Wu interleaved), EPI 3)
    h = mm_epi(act_quant(act), unpack(Wd), EPI 2, res=h)

epilogue="row" is the ablation that keeps INT32 GEMM outputs and applies scales, residuals, SwiGLU and the q/k norms in row
kernels (e2e/fused_qwen3.py:237-288).  With overlap=True the 4-bit -> INT8 decode of the next weight runs on a side stream
under the current GEMM.  rot=True / "down" quantizes rotated inputs (rot_quant) for packs made in the rotated basis.
"""
import numpy as np
import torch

from . import fused_dense as FD
from . import host_model as HM
from . import packed_io
from . import sc_format as F
from . import sc_kernels as S
from .w4a8 import PackedWeight

GROUPS = {"qkv": ["self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj"], "o": ["self_attn.o_proj"],
          "gu": ["mlp.gate_proj", "mlp.up_proj"], "down": ["mlp.down_proj"]}


def _get(layer, path):
    for p in path.split("."):
        layer = getattr(layer, p)
    return layer


def pack_model(model, cache_path=None, fmt=F.DEFAULT, on_device=False):
    """Packs every transformer-block linear; returns {"layers.{i}.{path}": (codes, bcodes, wscale)}, cached as one safetensors
    file when cache_path is given (e2e/w4a8_mlx.py:176-196, with 2-bit block codes as e2e/pack_format.py:83-109).  NumPy
    arrays by default; on_device=True keeps the quantizer's CUDA tensors (no host copies; same bits)."""
    import os
    if cache_path and os.path.exists(cache_path):
        return packed_io.load_packed(cache_path, fmt)
    out = {}
    for i, layer in enumerate(model.model.layers):
        for g in GROUPS.values():
            for path in g:
                w = _get(layer, path).weight.detach()
                if on_device:
                    out[f"layers.{i}.{path}"] = F.quantize_device(w.contiguous(), fmt, want_qw=False)[:3]
                else:
                    out[f"layers.{i}.{path}"] = F.quantize(w.to("cpu", torch.float64).numpy(), fmt)[:3]
    if cache_path:
        packed_io.save_packed(cache_path, {k: tuple(t.cpu().numpy() if torch.is_tensor(t) else t for t in v)
                                           for k, v in out.items()})
    return out


def load_packed(cache_path, n_layers, fmt=F.DEFAULT):
    """Per-linear packed weights from a cache file in either stored layout (e2e/fused_qwen3.py:62-73)."""
    flat = packed_io.load_packed(cache_path, fmt)
    return {f"layers.{i}.{p}": flat[f"layers.{i}.{p}"] for i in range(n_layers) for g in GROUPS.values() for p in g}


def tiles_for(M):
    """The reference tunes Metal tiles per shape here (e2e/fused_qwen3.py:76-80); the tcgen05 GEMM picks its own N tile."""
    return {"qkv": None, "o": None, "gu": None, "down": None}


class FusedQwen3:
    def __init__(self, model, packed, resident=False, overlap=True, epilogue="gemm", compiled=True, fmt=None, rot=False,
                 fuse_rope=True):
        """model: host_model.CausalLM on the GPU; packed: {"layers.{i}.{path}": (codes, bcodes, wscale)}.  resident keeps the
        INT8 operands decoded; fuse_rope=False applies the rotary embedding and the cache append with torch ops instead of
        inside the q/k/v kernel.  `compiled` is accepted for signature compatibility (there is no tracing compiler here)."""
        # rot: inputs rotated before INT8 (sc_kernels.rot_quant) for weights packed in the rotated basis; rot="down": only the
        # down projection's input (e2e/fused_qwen3.py:88-90).  Producing such packs (GPTQ in the rotated basis) is not part
        # of this library; they load through packed_io like any other pack.
        self.rot, self._signs = rot, {}
        assert epilogue in ("gemm", "row")
        self.fmt = fmt if fmt is not None else F.Format()
        S.set_format(self.fmt)
        self.model, self.args = model, model.args
        self.epilogue, self.resident, self.fuse_rope = epilogue, resident, fuse_rope
        self.eps = self.args.rms_norm_eps
        dev = model.model.embed_tokens.weight.device
        perm = {"gu": S.interleave_gate_up(self.args.intermediate_size)} if epilogue == "gemm" else {}
        self.layers = []
        for i, layer in enumerate(model.model.layers):
            ws = {g: PackedWeight([packed[f"layers.{i}.{p}"] for p in paths], perm.get(g), resident, dev)
                  for g, paths in GROUPS.items()}
            self.layers.append((layer, ws))
        for layer in model.model.layers:                      # the block linears are replaced: drop the bf16 weights
            for g in GROUPS.values():
                for path in g:
                    parent, name = path.split(".")
                    setattr(getattr(layer, parent), name, None)
        self.seq = [ws[g].entry() for _, ws in self.layers for g in GROUPS]
        self.ring = None if resident else FD.DecodeRing(max(e[3] * e[4] for e in self.seq), dev, overlap)
        self.inv_freq = S.rope_inv_freq(self.args.head_dim, self.args.rope_theta, dev)
        self.rope_cs = S.rope_table(self.inv_freq, 16384)          # cos / sin of the first positions, read by the q/k/v kernel
        self.record, self.record_layers = None, ()
        self.sdpa = HM.sdpa                                   # (q, k, v, scale, causal) -> [L, hq * d]; replaceable

    # ---- pieces -------------------------------------------------------------------------------------------------------
    def weight_bytes(self):
        return sum(w.nbytes() for _, ws in self.layers for w in ws.values())

    def signs(self, K):
        if K not in self._signs:
            self._signs[K] = S.rot_signs(K, self.inv_freq.device)
        return self._signs[K]

    def rms_q(self, h, nw, Mp=None):
        if self.rot is not True:
            return S.rmsnorm_quant(h, nw, self.eps, Mp)
        xn = S.rmsnorm_quant_n(h, nw, self.eps, Mp)[2]
        return S.rot_quant(xn[:h.shape[0]], self.signs(h.shape[1]), Mp)

    def act_q(self, x, Mp=None, nt=256, down=False):
        if not (self.rot is True or (self.rot == "down" and down)):
            return S.act_quant(x, Mp)
        return S.rot_quant(x, self.signs(x.shape[1]), Mp)

    def _rec(self, i, g, x, xq, wq, acc):
        if self.record is not None and i in self.record_layers:
            self.record[(i, g)] = (x, xq, wq.clone(), acc)

    def _w(self, g):
        if self.ring is None:
            return self.layers[g // 4][1][list(GROUPS)[g % 4]].wq
        return self.ring.weight(g)

    def _done(self, g):
        if self.ring is not None:
            self.ring.released(g)

    def _qkv(self, at, c, src, xs, ws, L):
        a = self.args
        hq, hk, d = a.num_attention_heads, a.num_key_value_heads, a.head_dim
        kw = dict(rope=(self.inv_freq, c.offset, self.rope_cs), cache=c) if self.fuse_rope else {}
        if src.dtype == torch.int32:
            q, k, v = S.qkv_epilogue_headnorm(src, xs, ws, at.q_norm.weight, at.k_norm.weight, self.eps, L, hq, hk, d, **kw)
        else:
            q, k, v = S.qkv_headnorm_y(src, at.q_norm.weight, at.k_norm.weight, self.eps, L, hq, hk, d, **kw)
        if self.fuse_rope:
            c.offset += L
        else:
            q, k = HM.rope(q, self.inv_freq, c.offset), HM.rope(k, self.inv_freq, c.offset)
            k, v = c.update_and_fetch(k, v)
        return q, k, v

    def _attention(self, at, c, src, xs, ws, L):
        q, k, v = self._qkv(at, c, src, xs, ws, L)
        return self.sdpa(q, k, v, at.scale, True)

    # ---- prefill ------------------------------------------------------------------------------------------------------
    @torch.no_grad()
    def hidden(self, ids, cache):
        """Final normed hidden states [1, L, D] for prompt ids [1, L] (prefill into a fresh or offset cache)."""
        S.set_format(self.fmt)
        h = self.model.model.embed_tokens(ids)[0]
        L = h.shape[0]
        Mp = S.pad_rows(L)
        if Mp != L:
            h = torch.nn.functional.pad(h, (0, 0, 0, Mp - L))
        h = h.contiguous()
        if self.ring is not None:
            self.ring.begin(self.seq)
        h = (self._blocks_gemm_epi if self.epilogue == "gemm" else self._blocks_row_epi)(h, cache, L, Mp)
        if self.ring is not None:
            self.ring.end()
        xn = S.rmsnorm_quant_n(h, self.model.model.norm.weight, self.eps, Mp)[2]
        return xn[:L][None]

    def _blocks_gemm_epi(self, h, cache, L, Mp):
        nl = len(self.layers)
        xq, xs = self.rms_q(h, self.layers[0][0].input_layernorm.weight, Mp)
        for i, (layer, ws) in enumerate(self.layers):
            at, g = layer.self_attn, 4 * i
            wq = self._w(g)
            y = S.mm_epi(xq, wq, xs, ws["qkv"].wscale, 1)
            self._done(g)
            self._rec(i, "qkv", h, xq, wq, None)
            o = self._attention(at, cache[i], y, None, None, L)
            xq, xs = self.act_q(o, Mp)
            wq = self._w(g + 1)
            self._rec(i, "o", o, xq, wq, None)
            h = S.mm_epi(xq, wq, xs, ws["o"].wscale, 2, res=h)
            self._done(g + 1)
            xq, xs = self.rms_q(h, layer.post_attention_layernorm.weight)
            wq = self._w(g + 2)
            self._rec(i, "gu", h, xq, wq, None)
            act = S.mm_epi(xq, wq, xs, ws["gu"].wscale, 3)
            self._done(g + 2)
            xq, xs = self.act_q(act, down=True)
            wq = self._w(g + 3)
            self._rec(i, "down", act, xq, wq, None)
            h = S.mm_epi(xq, wq, xs, ws["down"].wscale, 2, res=h)
            self._done(g + 3)
            if i + 1 < nl:
                xq, xs = self.rms_q(h, self.layers[i + 1][0].input_layernorm.weight)
        return h

    def _blocks_row_epi(self, h, cache, L, Mp):
        nl = len(self.layers)
        xq, xs = self.rms_q(h, self.layers[0][0].input_layernorm.weight, Mp)
        for i, (layer, ws) in enumerate(self.layers):
            at, g = layer.self_attn, 4 * i
            wq = self._w(g)
            acc = S.mm_i8_i32(xq, wq)
            self._done(g)
            self._rec(i, "qkv", h, xq, wq, acc)
            o = self._attention(at, cache[i], acc, xs, ws["qkv"].wscale, L)
            xq, xs = self.act_q(o, Mp)
            wq = self._w(g + 1)
            acc = S.mm_i8_i32(xq, wq)
            self._done(g + 1)
            self._rec(i, "o", o, xq, wq, acc)
            h, xq, xs = S.res_norm_quant(acc, xs, ws["o"].wscale, h, layer.post_attention_layernorm.weight, self.eps)
            wq = self._w(g + 2)
            acc = S.mm_i8_i32(xq, wq)
            self._done(g + 2)
            self._rec(i, "gu", h, xq, wq, acc)
            xq, xs = S.swiglu_quant(acc, xs, ws["gu"].wscale)
            wq = self._w(g + 3)
            acc = S.mm_i8_i32(xq, wq)
            self._done(g + 3)
            self._rec(i, "down", None, xq, wq, acc)
            if i + 1 < nl:
                h, xq, xs = S.res_norm_quant(acc, xs, ws["down"].wscale, h,
                                             self.layers[i + 1][0].input_layernorm.weight, self.eps)
            else:
                h = S.res_epilogue(acc, xs, ws["down"].wscale, h)
        return h

    def make_cache(self, capacity=4096):
        return HM.make_prompt_cache(self.model, capacity)

    def logits(self, h):
        return self.model.head(h)

    def __call__(self, ids, cache=None):
        """Logits for every position."""
        cache = cache if cache is not None else self.make_cache(max(ids.shape[1], 1))
        return self.logits(self.hidden(ids, cache))


def load_fused(model, cache_path=None, **kw):
    """Packs (or loads the cached pack of) a host_model.CausalLM and wraps it (e2e/fused_qwen3.py:312-337 without the
    checkpoint download)."""
    return FusedQwen3(model, pack_model(model, cache_path), **kw)
