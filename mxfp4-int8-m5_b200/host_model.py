"""Torch containers for the decoder checkpoints the fused W4A8 paths wrap, with the attribute layout of the mlx_lm models
the reference wires into (model.model.layers[i].self_attn.q_proj, .mlp.gate_proj / .mlp.switch_mlp, ...; see
e2e/fused_qwen3.py:82-118 and e2e/fused_olmoe.py:132-176), plus what surrounds the W4A8 linears in a block: RMSNorm in
MLX's rounding order, half-split rotary embedding, a preallocated KV cache and scaled-dot-product attention (torch's).

`CausalLM.forward` is the unfused path: every linear is whatever module sits in the tree (a bf16 torch Linear, or a
W4A8Linear after apply_w4a8), as in e2e/w4a8_mlx.py:197-207.
"""
from dataclasses import dataclass

import torch
import torch.nn.functional as TF

from . import sc_kernels as S


@dataclass
class ModelArgs:
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    rms_norm_eps: float = 1e-6
    rope_theta: float = 1e6
    vocab_size: int = 32000
    tie_word_embeddings: bool = True
    num_experts: int = 0
    num_experts_per_tok: int = 0
    norm_topk_prob: bool = False
    model_type: str = "qwen3"


QWEN3_1_7B = ModelArgs(2048, 6144, 28, 16, 8, 128, 1e-6, 1e6, 151936, True)
OLMOE_1B_7B = ModelArgs(2048, 1024, 16, 16, 16, 128, 1e-5, 1e4, 50304, False, 64, 8, False, "olmoe")

LINEARS = ["self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj", "self_attn.o_proj",
           "mlp.gate_proj", "mlp.up_proj", "mlp.down_proj"]


class RMSNorm(torch.nn.Module):
    """w * T(x * rsqrt(mean(x^2) + eps)): the product x * inv is rounded to the activation type before the weight
    multiplies it, the order of MLX's rms_norm that the fused row kernels replicate."""

    def __init__(self, dims, eps):
        super().__init__()
        self.weight = torch.nn.Parameter(torch.ones(dims, dtype=torch.bfloat16), requires_grad=False)
        self.eps = eps

    def forward(self, x):
        xf = x.float()
        inv = torch.rsqrt(xf.double().pow(2).mean(-1, keepdim=True).float() + self.eps)
        return self.weight * (xf * inv).to(x.dtype)


def rope(x, inv_freq, offset=0):
    """Half-split rotary embedding of x [..., L, d] at positions offset.. (mlx.nn.RoPE(traditional=False))."""
    L, d = x.shape[-2], x.shape[-1]
    ang = torch.arange(offset, offset + L, device=x.device, dtype=torch.float32)[:, None] * inv_freq[None, :]
    c, s = torch.cos(ang.double()).float(), torch.sin(ang.double()).float()
    x1, x2 = x[..., :d // 2].float(), x[..., d // 2:].float()
    return torch.cat([x1 * c - x2 * s, x1 * s + x2 * c], -1).to(x.dtype)


class KVCache:
    """Keys and values of one layer in preallocated [heads, capacity, d] tensors; `offset` positions are filled."""

    def __init__(self, heads, d, capacity, device="cuda", dtype=torch.bfloat16):
        self.k = torch.empty((heads, capacity, d), dtype=dtype, device=device)
        self.v = torch.empty_like(self.k)
        self.offset = 0

    def update_and_fetch(self, k, v):
        L = k.shape[-2]
        assert self.offset + L <= self.k.shape[1], "KV cache capacity exceeded"
        self.k[:, self.offset:self.offset + L] = k.reshape(self.k.shape[0], L, -1)
        self.v[:, self.offset:self.offset + L] = v.reshape(self.k.shape[0], L, -1)
        self.offset += L
        return self.k[:, :self.offset], self.v[:, :self.offset]


def sdpa(q, k, v, scale, causal):
    """q [hq, L, d], k / v [hk, T, d] (T >= L: the last L keys are the queries' own positions) -> [L, hq * d]."""
    hq, L, d = q.shape
    hk, T = k.shape[0], k.shape[1]
    mask = None
    is_causal = bool(causal and L > 1 and T == L)
    if causal and L > 1 and T != L:
        mask = torch.ones(L, T, dtype=torch.bool, device=q.device).tril(T - L)
    o = TF.scaled_dot_product_attention(q[None], k[None], v[None], attn_mask=mask, is_causal=is_causal, scale=scale,
                                        enable_gqa=hq != hk)
    return o[0].transpose(0, 1).reshape(L, hq * d)


def sdpa_f64(q, k, v, scale, causal):
    """The same attention in float64 with a single rounding at the output: a slow, kernel-independent form for checks."""
    hq, L, d = q.shape
    hk, T = k.shape[0], k.shape[1]
    kk, vv = (t.double().repeat_interleave(hq // hk, 0) for t in (k, v))
    s = torch.einsum("hld,htd->hlt", q.double(), kk) * scale
    if causal:
        s.masked_fill_(~torch.ones(L, T, dtype=torch.bool, device=q.device).tril(T - L), float("-inf"))
    o = torch.einsum("hlt,htd->hld", torch.softmax(s, -1), vv)
    return o.transpose(0, 1).reshape(L, hq * d).to(q.dtype)


def _linear(i, o):
    lin = torch.nn.Linear(i, o, bias=False, dtype=torch.bfloat16)
    lin.weight.requires_grad_(False)
    return lin


class Attention(torch.nn.Module):
    def __init__(self, a):
        super().__init__()
        D, hq, hk, d = a.hidden_size, a.num_attention_heads, a.num_key_value_heads, a.head_dim
        self.hq, self.hk, self.d, self.scale = hq, hk, d, d ** -0.5
        self.full_norm = a.model_type == "olmoe"
        self.q_proj, self.k_proj, self.v_proj, self.o_proj = _linear(D, hq * d), _linear(D, hk * d), _linear(D, hk * d), _linear(hq * d, D)
        self.q_norm = RMSNorm(hq * d if self.full_norm else d, a.rms_norm_eps)
        self.k_norm = RMSNorm(hk * d if self.full_norm else d, a.rms_norm_eps)
        self.register_buffer("inv_freq", S.rope_inv_freq(d, a.rope_theta, None), persistent=False)

    def forward(self, x, cache):
        L = x.shape[0]
        q, k, v = self.q_proj(x), self.k_proj(x), self.v_proj(x)
        if self.full_norm:
            q, k = self.q_norm(q), self.k_norm(k)
        q = q.reshape(L, self.hq, self.d).transpose(0, 1)
        k = k.reshape(L, self.hk, self.d).transpose(0, 1)
        v = v.reshape(L, self.hk, self.d).transpose(0, 1)
        if not self.full_norm:
            q, k = self.q_norm(q), self.k_norm(k)
        q, k = rope(q, self.inv_freq, cache.offset), rope(k, self.inv_freq, cache.offset)
        k, v = cache.update_and_fetch(k, v)
        return self.o_proj(sdpa(q, k, v, self.scale, True))


class MLP(torch.nn.Module):
    def __init__(self, a):
        super().__init__()
        D, F = a.hidden_size, a.intermediate_size
        self.gate_proj, self.up_proj, self.down_proj = _linear(D, F), _linear(D, F), _linear(F, D)

    def forward(self, x):
        return self.down_proj(TF.silu(self.gate_proj(x)) * self.up_proj(x))


class _Stacked(torch.nn.Module):
    def __init__(self, E, o, i):
        super().__init__()
        self.weight = torch.nn.Parameter(torch.empty((E, o, i), dtype=torch.bfloat16), requires_grad=False)


class SwitchMLP(torch.nn.Module):
    """Expert weights stacked [E, out, in] per projection (mlx_lm's switch_mlp layout)."""

    def __init__(self, a):
        super().__init__()
        E, D, F = a.num_experts, a.hidden_size, a.intermediate_size
        self.gate_proj, self.up_proj, self.down_proj = _Stacked(E, F, D), _Stacked(E, F, D), _Stacked(E, D, F)


class MoeMLP(torch.nn.Module):
    def __init__(self, a):
        super().__init__()
        self.k, self.norm_topk = a.num_experts_per_tok, a.norm_topk_prob
        self.gate = _linear(a.hidden_size, a.num_experts)
        self.switch_mlp = SwitchMLP(a)

    def forward(self, x):
        rw = torch.softmax(self.gate(x).float(), dim=1).to(x.dtype)
        scores, inds = torch.topk(rw, self.k, dim=-1)
        if self.norm_topk:
            scores = scores / scores.sum(-1, keepdim=True)
        sw, out = self.switch_mlp, torch.zeros_like(x)
        for e in inds.unique().tolist():
            t, j = (inds == e).nonzero(as_tuple=True)
            xe = x[t]
            ye = (TF.silu(xe @ sw.gate_proj.weight[e].T) * (xe @ sw.up_proj.weight[e].T)) @ sw.down_proj.weight[e].T
            out.index_add_(0, t, ye * scores[t, j][:, None])
        return out


class Layer(torch.nn.Module):
    def __init__(self, a):
        super().__init__()
        self.self_attn = Attention(a)
        self.mlp = MoeMLP(a) if a.num_experts else MLP(a)
        self.input_layernorm = RMSNorm(a.hidden_size, a.rms_norm_eps)
        self.post_attention_layernorm = RMSNorm(a.hidden_size, a.rms_norm_eps)

    def forward(self, h, cache):
        h = h + self.self_attn(self.input_layernorm(h), cache)
        return h + self.mlp(self.post_attention_layernorm(h))


class Inner(torch.nn.Module):
    def __init__(self, a):
        super().__init__()
        self.embed_tokens = torch.nn.Embedding(a.vocab_size, a.hidden_size, dtype=torch.bfloat16)
        self.embed_tokens.weight.requires_grad_(False)
        self.layers = torch.nn.ModuleList(Layer(a) for _ in range(a.num_hidden_layers))
        self.norm = RMSNorm(a.hidden_size, a.rms_norm_eps)


class CausalLM(torch.nn.Module):
    """Qwen3-style dense or OLMoE-style mixture-of-experts decoder (args.num_experts > 0)."""

    def __init__(self, args):
        super().__init__()
        self.args = args
        self.model = Inner(args)
        self.lm_head = None if args.tie_word_embeddings else _linear(args.hidden_size, args.vocab_size)

    def head(self, h):
        return TF.linear(h, self.model.embed_tokens.weight) if self.lm_head is None else self.lm_head(h)

    def forward(self, ids, cache=None):
        """ids int [1, L] -> logits [1, L, V]; prefill into a fresh or offset cache."""
        cache = cache if cache is not None else make_prompt_cache(self, ids.shape[1])
        h = self.model.embed_tokens(ids)[0]
        for layer, c in zip(self.model.layers, cache):
            h = layer(h, c)
        return self.head(self.model.norm(h)[None])

    @torch.no_grad()
    def init_random(self, seed=0, scale=0.02):
        """Seeded synthetic weights of the architecture (no checkpoint is read), generated on the parameters' device."""
        dev = self.model.embed_tokens.weight.device
        g = torch.Generator(device=dev).manual_seed(seed)
        for name, p in self.named_parameters():
            r = torch.randn(p.shape, generator=g, device=dev, dtype=torch.float32)
            if name.endswith("norm.weight") or "layernorm" in name:
                p.copy_((1.0 + 0.1 * r).to(p.dtype))
            else:
                p.copy_((scale * r).to(p.dtype))
        return self

    @torch.no_grad()
    def load_hf_state_dict(self, sd):
        """Hugging Face key names (model.layers.{i}.mlp.experts.{e}.gate_proj.weight are stacked into switch_mlp)."""
        own = dict(self.named_parameters())
        for k, p in own.items():
            if ".switch_mlp." in k:
                pre, proj = k.split(".switch_mlp.")
                proj = proj[:-len(".weight")]
                p.copy_(torch.stack([sd[f"{pre}.experts.{e}.{proj}.weight"] for e in range(p.shape[0])]).to(p.dtype))
            else:
                p.copy_(sd[k].to(p.dtype))
        return self


def make_prompt_cache(model, capacity, device=None):
    a = model.args
    device = device or model.model.embed_tokens.weight.device
    return [KVCache(a.num_key_value_heads, a.head_dim, capacity, device) for _ in model.model.layers]
