"""Fused SC-MXFP4 W4A8 prefill for OLMoE-style mixture-of-experts decoders: the torch counterpart of the reference's
FusedOlmoe (e2e/fused_olmoe.py:132-290) over libscmx.  Per block:

    y = mm_epi(xq, unpack(Wq|Wk|Wv), EPI 1);  q, k, v = qkv_fullnorm_y(y)  (+ rotary embedding, KV-cache append)
    o = sdpa(q, k, v);  h = mm_epi(act_quant(o), unpack(Wo), EPI 2, res=h)
    xq, xs, xn = rmsnorm_quant_n(h);  inds, scores = router(xn)            softmax / top-k on the device
    route_sort -> gather_rows -> moe_mm(gate|up, SwiGLU) -> act_quant -> moe_mm(down) -> moe_combine(+res, next norm + INT8)
"""
import os

import numpy as np
import torch

from . import host_model as HM
from . import packed_io
from . import sc_format as F
from . import sc_kernels as S
from . import sc_moe as M_
from .w4a8 import PackedWeight

ATTN = ["self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj", "self_attn.o_proj"]
EXPERTS = ["gate_proj", "up_proj", "down_proj"]


def pack_olmoe(model, cache_path=None, fmt=F.DEFAULT, on_device=False):
    """SC-MXFP4 of every attention linear and expert matrix; keys layers.{i}.{path} and layers.{i}.experts.{name}.{e}
    (e2e/fused_olmoe.py:102-129).  Returns {key: (codes, bcodes, wscale)} as NumPy, or with on_device=True as CUDA tensors
    (the experts of a layer are quantized in one call: the format is per output row, so the bits are the same)."""
    if cache_path and os.path.exists(cache_path):
        return packed_io.load_packed(cache_path, fmt)
    out = {}

    def q(w):
        if on_device:
            return F.quantize_device(w.contiguous(), fmt, want_qw=False)[:3]
        return F.quantize(w.to("cpu", torch.float64).numpy(), fmt)[:3]

    for i, layer in enumerate(model.model.layers):
        for path in ATTN:
            parent, name = path.split(".")
            out[f"layers.{i}.{path}"] = q(getattr(getattr(layer, parent), name).weight.detach())
        sw = layer.mlp.switch_mlp
        for name in EXPERTS:
            wt = getattr(sw, name).weight.detach()
            E, n, k = wt.shape
            c, b, s = q(wt.reshape(E * n, k))
            c, b, s = c.reshape(E, n * k // 8), b.reshape(E, n, -1), s.reshape(E, n)
            for e in range(E):
                out[f"layers.{i}.experts.{name}.{e}"] = (c[e], b[e], s[e])
    if cache_path:
        packed_io.save_packed(cache_path, {k: tuple(t.cpu().numpy() if torch.is_tensor(t) else t for t in v)
                                           for k, v in out.items()})
    return out


class FusedOlmoe:
    def __init__(self, model, flat, tile_gu=None, tile_d=None, bk=None, two_pass="auto", sort="count", compiled=True):
        """model: host_model.CausalLM (num_experts > 0) on the GPU; flat: pack_olmoe's dict.  two_pass=True decodes all
        experts to INT8 once per call and runs the grouped GEMM on that (moe_mm_i8); "auto": once the average expert has
        >= 256 rows (e2e/fused_olmoe.py:135-141).  The tile arguments are Metal tuning hints: accepted and ignored."""
        assert sort == "count"
        self.model, self.args = model, model.args
        a = self.args
        assert not a.norm_topk_prob
        self.eps, self.two_pass = a.rms_norm_eps, two_pass
        dev = model.model.embed_tokens.weight.device
        E, Fi = a.num_experts, a.intermediate_size
        perm = S.interleave_gate_up(Fi)
        idx = torch.as_tensor(perm, device=dev, dtype=torch.long)

        def cu(x, np_dtype):
            if isinstance(x, torch.Tensor):
                return x.to(dev)
            a = np.ascontiguousarray(np.asarray(x, np_dtype))
            return torch.from_numpy(a.view(np.int32) if np_dtype == np.uint32 else a).to(dev)

        self.layers = []
        for i, layer in enumerate(model.model.layers):
            parts = lambda p: flat[f"layers.{i}.{p}"]  # noqa: E731
            qkv = PackedWeight([parts(p) for p in ATTN[:3]], device=dev)
            o = PackedWeight([parts(ATTN[3])], device=dev)
            st = {}
            for n in EXPERTS:
                ps = [parts(f"experts.{n}.{e}") for e in range(E)]
                rows = int(ps[0][2].shape[0])
                st[n] = (torch.stack([cu(p[0], np.uint32).reshape(rows, -1) for p in ps]),
                         torch.stack([cu(p[1], np.uint8) for p in ps]), torch.stack([cu(p[2], np.float32) for p in ps]))
            g, u, d = st["gate_proj"], st["up_proj"], st["down_proj"]
            gu = tuple(torch.cat([a_, b_], 1)[:, idx].contiguous() for a_, b_ in zip(g, u))
            ex = dict(gu=(gu[0].reshape(E, -1), gu[1], gu[2]), down=(d[0].reshape(E, -1).contiguous(), d[1].contiguous(), d[2].contiguous()))
            self.layers.append((layer, dict(qkv=qkv, o=o), ex))
        self.perm_gu = perm
        for layer in model.model.layers:                      # drop the bf16 weights that the packed ones replace
            for path in ATTN:
                setattr(layer.self_attn, path.split(".")[1], None)
            layer.mlp.switch_mlp = None
        # Expert weights of the NEXT layer are decoded to INT8 on a side stream while the current layer runs (two rotating
        # buffer pairs), when the INT8 copy of one layer's experts is at most 1 GiB; the grouped GEMMs then read those
        # (moe_mm_i8).  Otherwise moe_mm decodes groups of experts between its own GEMM passes.
        F2, D = 2 * Fi, a.hidden_size
        self.prefetch = E * (F2 * D + D * Fi) <= (1 << 30)
        if self.prefetch:
            self.ring = [(torch.empty((E * F2, D), dtype=torch.int8, device=dev),
                          torch.empty((E * D, Fi), dtype=torch.int8, device=dev)) for _ in range(2)]
            self.side = torch.cuda.Stream(device=dev)
        self.inv_freq = S.rope_inv_freq(a.head_dim, a.rope_theta, dev)
        self.rope_cs = S.rope_table(self.inv_freq, 16384)          # cos / sin of the first positions, read by the q/k/v kernel
        self.record, self.record_layers = None, ()
        self.sdpa = HM.sdpa                                   # (q, k, v, scale, causal) -> [L, H * d]; replaceable

    def weight_bytes(self):
        n = 0
        for _, ws, ex in self.layers:
            n += ws["qkv"].nbytes() + ws["o"].nbytes()
            n += sum(t.numel() * t.element_size() for t in ex["gu"] + ex["down"])
        return n

    def route(self, layer, xn, M):
        """Router of the block on the normalized bf16 rows: softmax over experts then top-k (e2e/fused_olmoe.py:186-195)."""
        logits = torch.nn.functional.linear(xn[:M], layer.mlp.gate.weight)
        return M_.router_topk(logits.float(), self.args.num_experts_per_tok)

    def _decode_experts(self, i):
        """Layer i's experts -> INT8 in ring[i % 2] on the side stream; waits for the GEMMs that last read that pair."""
        a = self.args
        E, F2, D = a.num_experts, 2 * a.intermediate_size, a.hidden_size
        (cg, bg, _), (cd, bd, _) = self.layers[i][2]["gu"], self.layers[i][2]["down"]
        gu8, dn8 = self.ring[i % 2]
        with torch.cuda.stream(self.side):
            if i >= 2:
                self.side.wait_event(self._done[i - 2])
            S.unpack_i8(cg.reshape(-1), bg.reshape(E * F2, -1), E * F2, D, out=gu8)
            S.unpack_i8(cd.reshape(-1), bd.reshape(E * D, -1), E * D, F2 // 2, out=dn8)
            self._ready[i] = torch.cuda.Event()
            self._ready[i].record(self.side)

    def experts(self, ex, xq, xs, inds, L, decoded=None):
        """INT8 rows + routing -> (sorted expert outputs yd bf16 [R, D], pos).  decoded: (gu8, dn8) INT8 copies of this
        layer's experts when they were decoded ahead."""
        a = self.args
        k, E, F2, D = a.num_experts_per_tok, a.num_experts, 2 * a.intermediate_size, a.hidden_size
        R = L * k
        two_pass = self.two_pass if self.two_pass != "auto" else R // E >= 256
        pos, tok_p, e_sorted, off, tstart, maxt = M_.route_sort(inds, E, M_.TM)
        xq_s, xs_s = M_.gather_rows(xq, xs, tok_p, R)
        (cg, bg, sg), (cd, bd, sd) = ex["gu"], ex["down"]
        if decoded is not None:
            act = M_.moe_mm_i8(xq_s, R, decoded[0], sg, off, tstart, maxt, F2, 3, xs_s)
            xq2, xs2 = S.act_quant(act, R + M_.TM)
            yd = M_.moe_mm_i8(xq2, R, decoded[1], sd, off, tstart, maxt, D, 1, xs2)
            return yd, pos, (xq_s, xs_s, act, xq2, xs2, e_sorted)
        if two_pass:
            act = M_.moe_mm_i8(xq_s, R, M_.unpack_experts(cg, bg, F2, D), sg, off, tstart, maxt, F2, 3, xs_s)
        else:
            act = M_.moe_mm(xq_s, R, cg, bg, sg, off, tstart, maxt, F2, 3, xs_s)
        xq2, xs2 = S.act_quant(act, R + M_.TM)
        if two_pass:
            yd = M_.moe_mm_i8(xq2, R, M_.unpack_experts(cd, bd, D, F2 // 2), sd, off, tstart, maxt, D, 1, xs2)
        else:
            yd = M_.moe_mm(xq2, R, cd, bd, sd, off, tstart, maxt, D, 1, xs2)
        return yd, pos, (xq_s, xs_s, act, xq2, xs2, e_sorted)

    @torch.no_grad()
    def hidden(self, ids, cache):
        a = self.args
        H, d, D = a.num_attention_heads, a.head_dim, a.hidden_size
        h = self.model.model.embed_tokens(ids)[0]
        L = h.shape[0]
        Mp = S.pad_rows(L)
        if Mp != L:
            h = torch.nn.functional.pad(h, (0, 0, 0, Mp - L))
        h = h.contiguous()
        nl = len(self.layers)
        main = torch.cuda.current_stream()
        if self.prefetch:
            self._ready, self._done = [None] * nl, [None] * nl
            self.side.wait_stream(main)
            self._decode_experts(0)
        xq, xs = S.rmsnorm_quant(h, self.layers[0][0].input_layernorm.weight, self.eps, Mp)
        for i, (layer, ws, ex) in enumerate(self.layers):
            at, c = layer.self_attn, cache[i]
            if self.prefetch and i + 1 < nl:
                self._decode_experts(i + 1)                    # under this layer's attention and GEMMs
            wq, wo = ws["qkv"], ws["o"]
            y = S.mm_epi(xq, wq.unpack(), xs, wq.wscale, 1)
            q, kk, v = S.qkv_fullnorm_y(y, at.q_norm.weight, at.k_norm.weight, self.eps, L, H, d,
                                        rope=(self.inv_freq, c.offset, self.rope_cs), cache=c)
            c.offset += L
            o = self.sdpa(q, kk, v, at.scale, True)
            xq, xs = S.act_quant(o, Mp)
            h = S.mm_epi(xq, wo.unpack(), xs, wo.wscale, 2, res=h)
            xq, xs, xn = S.rmsnorm_quant_n(h, layer.post_attention_layernorm.weight, self.eps)
            inds, scores = self.route(layer, xn, L)
            if self.prefetch:
                main.wait_event(self._ready[i])
            yd, pos, rec = self.experts(ex, xq, xs, inds, L, self.ring[i % 2] if self.prefetch else None)
            if self.prefetch:
                self._done[i] = torch.cuda.Event()
                self._done[i].record(main)
            nn = self.layers[i + 1][0].input_layernorm.weight if i + 1 < nl else self.model.model.norm.weight
            h_in = h
            h, xq, xs = M_.moe_combine(yd, pos, scores, h, nn, self.eps, L)
            if self.record is not None and i in self.record_layers:
                self.record[(i, "experts")] = (h_in, xn, inds, scores, yd, pos, *rec)
        if self.prefetch:
            main.wait_stream(self.side)
        xn = S.rmsnorm_quant_n(h, self.model.model.norm.weight, self.eps, Mp)[2]
        return xn[:L][None]

    def make_cache(self, capacity=4096):
        return HM.make_prompt_cache(self.model, capacity)

    def logits(self, h):
        return self.model.head(h)

    def __call__(self, ids, cache=None):
        cache = cache if cache is not None else self.make_cache(max(ids.shape[1], 1))
        return self.logits(self.hidden(ids, cache))


def load_fused_olmoe(model, cache_path=None, **kw):
    return FusedOlmoe(model, pack_olmoe(model, cache_path), **kw)
