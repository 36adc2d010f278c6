"""Batch-1 decode (token generation) with W4A8 GEMVs that read the packed 4-bit weights directly: the torch counterpart of
the reference's DecodeQwen3 / DecodeOlmoe (e2e/decode.py:29-165) over libscmx.  The linears compute the same function as
the prefill path (same INT8 activations, exact integer totals, same epilogues); attention is torch's at L = 1.

fuse_prologue selects where the per-token INT8 of a GEMV input is computed in the reference (inside the GEMV or in a row
kernel); here both forms run the row kernel followed by the GEMV and give the same values, so the argument only keeps the
signature."""
import torch

from . import host_model as HM
from . import sc_decode as G
from . import sc_kernels as S
from . import sc_moe as M_


def _head_fn(model, head):
    src = model if head == "model" else head
    return src.head


class DecodeQwen3:
    """Built from a FusedQwen3 with epilogue="gemm" (gate/up rows interleaved for the SwiGLU epilogue)."""

    def __init__(self, fused, head="model", compiled=True, fuse_prologue=None, act_tile=None):
        assert fused.epilogue == "gemm"
        self.f, self.model, self.args = fused, fused.model, fused.args
        self.head = _head_fn(fused.model, head)

    @torch.no_grad()
    def step(self, tok, cache):
        """tok int [1, 1] -> logits [1, 1, V]; appends one position to the cache."""
        f, a = self.f, self.args
        S.set_format(f.fmt)
        hq, hk, d, eps = a.num_attention_heads, a.num_key_value_heads, a.head_dim, f.eps
        h = self.model.model.embed_tokens(tok)[0]             # [1, D]
        for i, (layer, ws) in enumerate(f.layers):
            at, c = layer.self_attn, cache[i]
            w = ws["qkv"]
            xq, xs = S.rmsnorm_quant(h, layer.input_layernorm.weight, eps, 1)
            y = G.gemv(xq, w.codes, w.bcodes, xs, w.wscale, w.N, 1)
            q, k, v = S.qkv_headnorm_y(y[None], at.q_norm.weight, at.k_norm.weight, eps, 1, hq, hk, d,
                                       rope=(f.inv_freq, c.offset), cache=c)
            c.offset += 1
            o = f.sdpa(q, k, v, at.scale, False)
            wo, wg, wd = ws["o"], ws["gu"], ws["down"]
            h = G.gemv(o, wo.codes, wo.bcodes, None, wo.wscale, wo.N, 2, res=h, pro=1)[None]
            xq, xs = S.rmsnorm_quant(h, layer.post_attention_layernorm.weight, eps, 1)
            act = G.gemv(xq, wg.codes, wg.bcodes, xs, wg.wscale, wg.N, 3)
            h = G.gemv(act[None], wd.codes, wd.bcodes, None, wd.wscale, wd.N, 2, res=h, pro=1)[None]
        return self.head(self.model.model.norm(h)[None])


class DecodeOlmoe:
    """Built from a FusedOlmoe: the expert GEMVs gather the top-k experts' rows themselves."""

    def __init__(self, fused, head="model", compiled=True, fuse_prologue=False, o_tile=None):
        self.f, self.model, self.args = fused, fused.model, fused.args
        self.head = _head_fn(fused.model, head)
        assert not self.args.norm_topk_prob
        self.pos = torch.arange(self.args.num_experts_per_tok, dtype=torch.int32, device=fused.inv_freq.device)

    @torch.no_grad()
    def step(self, tok, cache):
        f, a = self.f, self.args
        H, d, D, eps = a.num_attention_heads, a.head_dim, a.hidden_size, f.eps
        F2, k = 2 * a.intermediate_size, a.num_experts_per_tok
        h = self.model.model.embed_tokens(tok)[0]
        for i, (layer, ws, ex) in enumerate(f.layers):
            at, c = layer.self_attn, cache[i]
            w, wo = ws["qkv"], ws["o"]
            xq, xs = S.rmsnorm_quant(h, layer.input_layernorm.weight, eps, 1)
            y = G.gemv(xq, w.codes, w.bcodes, xs, w.wscale, 3 * H * d, 1)
            q, kk, v = S.qkv_fullnorm_y(y[None], at.q_norm.weight, at.k_norm.weight, eps, 1, H, d,
                                        rope=(f.inv_freq, c.offset), cache=c)
            c.offset += 1
            o = f.sdpa(q, kk, v, at.scale, False)
            h = G.gemv(o, wo.codes, wo.bcodes, None, wo.wscale, D, 2, res=h, pro=1)[None]
            pn = layer.post_attention_layernorm.weight
            xq, xs, xn = S.rmsnorm_quant_n(h, pn, eps, 1)     # the router needs the bf16 normalized row too
            inds, scores = f.route(layer, xn, 1)
            e = inds.reshape(-1)
            (cg, bg, sg), (cd, bd, sd) = ex["gu"], ex["down"]
            act = G.gemv(xq, cg, bg, xs, sg, F2, 3, eidx=e, xstride=0)            # [k, F]
            xq2, xs2 = S.act_quant(act, k)
            yd = G.gemv(xq2, cd, bd, xs2, sd, D, 1, eidx=e, xstride=1)            # [k, D]
            h = M_.moe_combine(yd, self.pos, scores, h, pn, eps, 1, quant=False)[0]
        return self.head(self.model.model.norm(h)[None])
