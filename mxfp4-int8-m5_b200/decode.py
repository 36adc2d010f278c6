"""Batch-1 decode (token generation) with W4A8 GEMVs that read the packed 4-bit weights directly: the torch counterpart of
the reference's DecodeQwen3 / DecodeOlmoe (e2e/decode.py:29-165) over libscmx.  The linears compute the same function as
the prefill path (same INT8 activations, exact integer totals, same epilogues).

Attention at L = 1 is the library's own decode-attention kernel (attention="kernel"), which reads the sequence length on
the device, or torch's (attention="torch").  With the kernel, a whole step - embedding, every layer, output head, argmax,
position counter - is captured in one CUDA graph (`generate`) and replayed per token; the reference reaches the same end
by mx.compile'ing the halves of a step (e2e/decode.py:31-33).

fuse_prologue selects where the per-token INT8 of a GEMV input is computed in the reference (inside the GEMV or in a row
kernel); here both forms run the row kernel followed by the GEMV and give the same values, so the argument only keeps the
signature."""
import torch

from . import sc_decode as G
from . import sc_kernels as S
from . import sc_moe as M_


def _head_fn(model, head):
    src = model if head == "model" else head
    return src.head


class _Decoder:
    def __init__(self, fused, head, attention):
        self.f, self.model, self.args = fused, fused.model, fused.args
        self.head = _head_fn(fused.model, head)
        a = self.args
        hq, hk, d = a.num_attention_heads, a.num_key_value_heads, a.head_dim
        if attention == "kernel" and not S.DecodeAttention.supports(hq, hk, d):
            attention = "torch"
        self.attention = attention
        self.attn = S.DecodeAttention(hq, hk, d, fused.inv_freq.device) if attention == "kernel" else None
        self._graph = None

    def _attend(self, at, c, q, k, v, pos_dev):
        if self.attn is not None:
            return self.attn(q, c, at.scale, n_pos=None if pos_dev is not None else c.offset + 1, pos_dev=pos_dev)
        assert pos_dev is None, "a device-side position needs attention='kernel'"
        return self.f.sdpa(q, k, v, at.scale, False)

    @torch.no_grad()
    def step(self, tok, cache):
        """tok int [1, 1] -> logits [1, 1, V]; appends one position to the cache."""
        logits = self._step(tok, cache, None)
        for c in cache:
            c.offset += 1
        return logits

    @torch.no_grad()
    def generate(self, tok, cache, n):
        """Greedy decoding of n tokens after `tok` (int [1, 1]) from one captured CUDA graph replayed n times.
        Returns int64 [n]; the cache advances by n positions."""
        assert self.attn is not None, "graph decoding needs attention='kernel'"
        dev = tok.device
        if self._graph is None or self._graph[0] is not cache:
            offsets = [c.offset for c in cache]
            # the warm-up run below writes the cache row at `pos`: point it at the row the first real step overwrites
            tok_buf = tok.reshape(1, 1).to(torch.long).clone()
            pos = torch.full((1,), offsets[0], dtype=torch.int32, device=dev)
            for c in cache:
                c.offset = 0                                   # rows and rotary positions come from `pos` on the device
            s = torch.cuda.Stream(device=dev)
            s.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(s):
                self._step(tok_buf, cache, pos)                # warm-up outside the capture (lazy initialisations)
                torch.cuda.synchronize()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=s):
                    logits = self._step(tok_buf, cache, pos)
                    tok_buf.copy_(logits[:, -1].argmax(-1, keepdim=True))
                    pos.add_(1)
            torch.cuda.current_stream().wait_stream(s)
            for c, o in zip(cache, offsets):
                c.offset = o
            self._graph = (cache, g, tok_buf, pos, logits)
        _, g, tok_buf, pos, _ = self._graph
        start = cache[0].offset
        assert start + n <= cache[0].k.shape[1], "KV cache capacity exceeded"
        tok_buf.copy_(tok.reshape(1, 1))
        pos.fill_(start)
        out = torch.empty(n, dtype=torch.long, device=dev)
        for i in range(n):
            g.replay()
            out[i:i + 1].copy_(tok_buf.reshape(1))
        for c in cache:
            c.offset = start + n
        return out


class DecodeQwen3(_Decoder):
    """Built from a FusedQwen3 with epilogue="gemm" (gate/up rows interleaved for the SwiGLU epilogue)."""

    def __init__(self, fused, head="model", compiled=True, fuse_prologue=None, act_tile=None, attention="kernel"):
        assert fused.epilogue == "gemm"
        super().__init__(fused, head, attention)

    def _step(self, tok, cache, pos_dev):
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
                                       rope=(f.inv_freq, c.offset, f.rope_cs), cache=c, pos_dev=pos_dev)
            o = self._attend(at, c, q, k, v, pos_dev)
            wo, wg, wd = ws["o"], ws["gu"], ws["down"]
            h = G.gemv(o, wo.codes, wo.bcodes, None, wo.wscale, wo.N, 2, res=h, pro=1)[None]
            xq, xs = S.rmsnorm_quant(h, layer.post_attention_layernorm.weight, eps, 1)
            act = G.gemv(xq, wg.codes, wg.bcodes, xs, wg.wscale, wg.N, 3)
            h = G.gemv(act[None], wd.codes, wd.bcodes, None, wd.wscale, wd.N, 2, res=h, pro=1)[None]
        xn = S.rmsnorm_quant_n(h, self.model.model.norm.weight, eps, 1)[2]
        return self.head(xn[None])


class DecodeOlmoe(_Decoder):
    """Built from a FusedOlmoe: the expert GEMVs gather the top-k experts' rows themselves."""

    def __init__(self, fused, head="model", compiled=True, fuse_prologue=False, o_tile=None, attention="kernel"):
        super().__init__(fused, head, attention)
        assert not self.args.norm_topk_prob
        self.pos = torch.arange(self.args.num_experts_per_tok, dtype=torch.int32, device=fused.inv_freq.device)

    def _step(self, tok, cache, pos_dev):
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
                                        rope=(f.inv_freq, c.offset, f.rope_cs), cache=c, pos_dev=pos_dev)
            o = self._attend(at, c, q, kk, v, pos_dev)
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
        xn = S.rmsnorm_quant_n(h, self.model.model.norm.weight, eps, 1)[2]
        return self.head(xn[None])
