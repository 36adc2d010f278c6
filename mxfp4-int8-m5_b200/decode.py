"""Batch-1 decode (token generation) with W4A8 GEMVs that read the packed 4-bit weights directly: the torch counterpart of
the reference's DecodeQwen3 / DecodeOlmoe (e2e/decode.py:29-165) over libscmx.  The linears compute the same function as
the prefill path (same INT8 activations, exact integer totals, same epilogues).

Attention at L = 1 is the library's own decode-attention kernel (attention="kernel"), which reads the sequence length on
the device, or torch's (attention="torch").  With the kernel, a whole step - embedding, every layer, output head, argmax,
position counter - is captured in one CUDA graph (`generate`) and replayed per token; the reference reaches the same end
by mx.compile'ing the halves of a step (e2e/decode.py:31-33).

fuse_prologue selects where the per-token INT8 of a GEMV input is computed in the reference (inside the GEMV or in a row
kernel); here both forms run the row kernel followed by the GEMV and give the same values, so the argument only keeps the
signature.

persistent=True (DecodeQwen3) runs all layers of a step as ONE cooperative kernel (scmx_decode_step_dense): the phases of a
layer are separated by grid-wide barriers instead of kernel boundaries, each CTA re-quantizes the activations it needs in
shared memory, and weight loads are issued ahead of the barriers.  Same bits as the chain of kernels; used where its limits
hold (head size 128, widths multiples of 1024 up to 6144) and attention="kernel"."""
import ctypes

import numpy as np
import torch

from . import _lib
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
        self._mk = None                                       # persistent-kernel state, built per cache

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

    def __init__(self, fused, head="model", compiled=True, fuse_prologue=None, act_tile=None, attention="kernel",
                 persistent=True):
        assert fused.epilogue == "gemm"
        super().__init__(fused, head, attention)
        a = self.args
        fits = lambda n: n % 1024 == 0 and n <= 6144  # noqa: E731
        self.persistent = bool(persistent and self.attn is not None and a.head_dim == 128 and fits(a.hidden_size)
                               and fits(a.intermediate_size) and fits(a.num_attention_heads * a.head_dim)
                               and a.num_attention_heads <= 32 and fused.fmt == type(fused.fmt)())

    def _persistent_state(self, cache):
        """Layer table (device pointers of the packed weights, norms and this cache's tensors) and scratch buffers."""
        if self._mk is not None and self._mk["cache"] is cache:
            return self._mk
        f, a = self.f, self.args
        dev = f.inv_freq.device
        table = (_lib.ScmxDecodeLayer * len(f.layers))()
        for i, (layer, ws) in enumerate(f.layers):
            t, at, c = table[i], layer.self_attn, cache[i]
            for j, g in enumerate(("qkv", "o", "gu", "down")):
                t.codes[j], t.bcodes[j], t.wscale[j] = ws[g].codes.data_ptr(), ws[g].bcodes.data_ptr(), ws[g].wscale.data_ptr()
            t.ln_in, t.ln_post = layer.input_layernorm.weight.data_ptr(), layer.post_attention_layernorm.weight.data_ptr()
            t.q_norm, t.k_norm = at.q_norm.weight.data_ptr(), at.k_norm.weight.data_ptr()
            t.k_cache, t.v_cache = c.k.data_ptr(), c.v.data_ptr()
        raw = np.frombuffer(ctypes.string_at(ctypes.addressof(table), ctypes.sizeof(table)), dtype=np.uint8).copy()
        hq, hk, d = a.num_attention_heads, a.num_key_value_heads, a.head_dim
        self._mk = dict(cache=cache, table=torch.from_numpy(raw).to(dev),
                        y=torch.empty((hq + 2 * hk) * d, dtype=torch.bfloat16, device=dev),
                        act=torch.empty(a.intermediate_size, dtype=torch.bfloat16, device=dev),
                        o=torch.empty(hq * d, dtype=torch.bfloat16, device=dev),
                        bar=torch.zeros(2, dtype=torch.int32, device=dev),
                        status=torch.zeros(1, dtype=torch.int32, device=dev),
                        pos=torch.zeros(1, dtype=torch.int32, device=dev))
        return self._mk

    def check_status(self):
        """Raises if a barrier of the persistent kernel timed out (synchronizes)."""
        if self._mk is not None:
            st = int(self._mk["status"].item())
            if st:
                raise _lib.ScmxError(f"persistent decode kernel gave up at barrier {st - 100}")

    def _step_persistent(self, tok, cache, pos_dev):
        f, a = self.f, self.args
        mk = self._persistent_state(cache)
        if pos_dev is None:
            pos_dev = mk["pos"]
            pos_dev.fill_(cache[0].offset)
        hq, hk, d = a.num_attention_heads, a.num_key_value_heads, a.head_dim
        h = self.model.model.embed_tokens(tok)[0].clone()     # [1, D]; the kernel updates it in place
        _lib.call("scmx_decode_step_dense", _lib.ptr(mk["table"]), len(f.layers), a.hidden_size, a.intermediate_size, hq, hk, d,
                  float(f.eps), float(f.layers[0][0].self_attn.scale), _lib.ptr(f.inv_freq), _lib.ptr(f.rope_cs),
                  f.rope_cs.shape[0], cache[0].k.shape[1], _lib.ptr(pos_dev), _lib.ptr(h), _lib.ptr(mk["y"]), _lib.ptr(mk["act"]),
                  _lib.ptr(mk["o"]), _lib.ptr(self.attn.part), self.attn.nsplit, _lib.ptr(self.attn.counters), _lib.ptr(mk["bar"]),
                  _lib.ptr(mk["status"]), _lib.stream())
        xn = S.rmsnorm_quant_n(h, self.model.model.norm.weight, f.eps, 1)[2]
        return self.head(xn[None])

    def _step(self, tok, cache, pos_dev):
        f, a = self.f, self.args
        S.set_format(f.fmt)
        if self.persistent:
            return self._step_persistent(tok, cache, pos_dev)
        hq, hk, d, eps = a.num_attention_heads, a.num_key_value_heads, a.head_dim, f.eps
        h = self.model.model.embed_tokens(tok)[0]             # [1, D]
        for i, (layer, ws) in enumerate(f.layers):
            at, c = layer.self_attn, cache[i]
            w = ws["qkv"]
            y = G.gemv(h, w.codes, w.bcodes, None, w.wscale, w.N, 1, pro=2, nw=layer.input_layernorm.weight, eps=eps)
            q, k, v = S.qkv_headnorm_y(y[None], at.q_norm.weight, at.k_norm.weight, eps, 1, hq, hk, d,
                                       rope=(f.inv_freq, c.offset, f.rope_cs), cache=c, pos_dev=pos_dev)
            o = self._attend(at, c, q, k, v, pos_dev)
            wo, wg, wd = ws["o"], ws["gu"], ws["down"]
            h = G.gemv(o, wo.codes, wo.bcodes, None, wo.wscale, wo.N, 2, res=h, pro=1)[None]
            act = G.gemv(h, wg.codes, wg.bcodes, None, wg.wscale, wg.N, 3, pro=2, nw=layer.post_attention_layernorm.weight,
                         eps=eps)
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
            y = G.gemv(h, w.codes, w.bcodes, None, w.wscale, 3 * H * d, 1, pro=2, nw=layer.input_layernorm.weight, eps=eps)
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
            yd = G.gemv(act, cd, bd, None, sd, D, 1, eidx=e, xstride=1, pro=1)    # [k, D], per-row INT8 in the prologue
            h = M_.moe_combine(yd, self.pos, scores, h, pn, eps, 1, quant=False)[0]
        xn = S.rmsnorm_quant_n(h, self.model.model.norm.weight, eps, 1)[2]
        return self.head(xn[None])
