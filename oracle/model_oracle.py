"""TEST INFRASTRUCTURE ONLY: CPU restatement (NumPy) of a whole decoder forward built from the oracle's functions, for
checking how the fused paths wire the W4A8 kernels into a model (e2e/fused_qwen3.py:209-235, e2e/fused_olmoe.py:211-276).
Nothing shipped imports this file.

Two modes over the same wiring:
  "w4a8"  - the fused chain: INT8 activations, exact integer GEMMs on the decoded SC-MXFP4 weights, bf16 roundings where the
            reference rounds (scmx_oracle's functions), attention in float64 rounded to bf16 at its output;
  "float" - the same graph in float64 on given real-valued weights, no quantization or rounding: comparable with any
            standard implementation of the architecture (tests compare it with the Hugging Face models on CPU).

Parity unpinned for the parts outside the W4A8 kernels (rotary embedding, attention, router): the reference delegates
them to MLX, which is not available here; the "float" mode pins their wiring to the Hugging Face implementations instead.

Weights: dict of NumPy arrays
  embed [V, D], norm [D], lm_head [V, D] (absent when tied),
  layers.{i}.input_layernorm / post_attention_layernorm [D], layers.{i}.q_norm / k_norm,
  float mode: layers.{i}.self_attn.{q,k,v,o}_proj, layers.{i}.mlp.{gate,up,down}_proj [out, in];
              MoE: layers.{i}.gate [E, D], layers.{i}.experts.{gate_proj|up_proj|down_proj}.{e}
  w4a8 mode: `packed` = {"layers.{i}.<path>": (codes, bcodes, wscale)} under the same names.
"""
import numpy as np

try:
    from . import scmx_oracle as O
except ImportError:                      # imported with the oracle directory itself on sys.path
    import scmx_oracle as O

ATTN = ["self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj"]


def _attention(q, k, v, scale, offset=0):
    """q [hq, L, d], k / v [hk, T, d], causal with the queries at positions offset.. -> [L, hq * d] (float64)."""
    hq, L, d = q.shape
    hk, T = k.shape[0], k.shape[1]
    rep = hq // hk
    out = np.empty((L, hq, d), np.float64)
    mask = np.arange(T)[None, :] > (offset + np.arange(L))[:, None]
    for h in range(hq):
        s = (q[h].astype(np.float64) @ k[h // rep].astype(np.float64).T) * scale
        s[mask] = -np.inf
        s = np.exp(s - s.max(1, keepdims=True))
        out[:, h] = (s / s.sum(1, keepdims=True)) @ v[h // rep].astype(np.float64)
    return out.reshape(L, hq * d)


def _rms_float(x, w, eps):
    return x / np.sqrt((x ** 2).mean(-1, keepdims=True) + eps) * w


def _rope_float(x, inv_freq, offset):
    L, d = x.shape[1], x.shape[2]
    ang = np.arange(offset, offset + L, dtype=np.float64)[:, None] * inv_freq.astype(np.float64)[None]
    c, s = np.cos(ang)[None], np.sin(ang)[None]
    x1, x2 = x[..., :d // 2], x[..., d // 2:]
    return np.concatenate([x1 * c - x2 * s, x1 * s + x2 * c], -1)


def forward_float(W, args, ids):
    """Logits [L, V] in float64 for token ids [L]."""
    a = args
    hq, hk, d, D = a.num_attention_heads, a.num_key_value_heads, a.head_dim, a.hidden_size
    full = a.model_type == "olmoe"
    inv_freq = O.rope_inv_freq(d, a.rope_theta)
    L = len(ids)
    h = W["embed"][np.asarray(ids)].astype(np.float64)
    for i in range(a.num_hidden_layers):
        p = f"layers.{i}."
        x = _rms_float(h, W[p + "input_layernorm"], a.rms_norm_eps)
        q, k, v = (x @ W[p + n].astype(np.float64).T for n in ATTN)
        if full:
            q, k = _rms_float(q, W[p + "q_norm"], a.rms_norm_eps), _rms_float(k, W[p + "k_norm"], a.rms_norm_eps)
        q, k, v = (t.reshape(L, -1, d).transpose(1, 0, 2) for t in (q, k, v))
        if not full:
            q, k = _rms_float(q, W[p + "q_norm"], a.rms_norm_eps), _rms_float(k, W[p + "k_norm"], a.rms_norm_eps)
        q, k = _rope_float(q, inv_freq, 0), _rope_float(k, inv_freq, 0)
        o = _attention(q, k, v, d ** -0.5)
        h = h + o @ W[p + "self_attn.o_proj"].astype(np.float64).T
        x = _rms_float(h, W[p + "post_attention_layernorm"], a.rms_norm_eps)
        silu = lambda g: g / (1 + np.exp(-g))  # noqa: E731
        if a.num_experts:
            lg = x @ W[p + "gate"].astype(np.float64).T
            pr = np.exp(lg - lg.max(1, keepdims=True))
            pr /= pr.sum(1, keepdims=True)
            inds = np.argsort(-pr, axis=1, kind="stable")[:, :a.num_experts_per_tok]
            y = np.zeros_like(h)
            for t in range(L):
                for e in inds[t]:
                    wg, wu, wd = (W[p + f"experts.{n}.{e}"].astype(np.float64) for n in ("gate_proj", "up_proj", "down_proj"))
                    y[t] += pr[t, e] * ((silu(x[t] @ wg.T) * (x[t] @ wu.T)) @ wd.T)
            h = h + y
        else:
            wg, wu, wd = (W[p + f"mlp.{n}"].astype(np.float64) for n in ("gate_proj", "up_proj", "down_proj"))
            h = h + (silu(x @ wg.T) * (x @ wu.T)) @ wd.T
    x = _rms_float(h, W["norm"], a.rms_norm_eps)
    return x @ W.get("lm_head", W["embed"]).astype(np.float64).T


def _decoded(packed, names, fmt):
    """Row concatenation of packed matrices -> (INT8 values [N, K] as int32, wscale [N])."""
    qs, ss = [], []
    for n in names:
        c, b, s = packed[n]
        N = np.asarray(s).shape[0]
        K = np.asarray(c).size * 8 // N
        qs.append(O.decode(np.asarray(c, np.uint32), np.asarray(b, np.uint8), N, K, fmt))
        ss.append(np.asarray(s, np.float32))
    return np.concatenate(qs), np.concatenate(ss)


def forward_w4a8(W, packed, args, ids, fmt=O.DEFAULT, trace=None):
    """Logits [L, V] (bf16 values as float32) of the fused W4A8 chain for token ids [L] into a fresh cache.  trace, when a
    dict, receives the residual stream after every block."""
    a = args
    hq, hk, d, D, Fi = a.num_attention_heads, a.num_key_value_heads, a.head_dim, a.hidden_size, a.intermediate_size
    full, eps = a.model_type == "olmoe", a.rms_norm_eps
    inv_freq = O.rope_inv_freq(d, a.rope_theta)
    perm = O.interleave_gate_up(Fi)
    L = len(ids)
    Mp = O.pad_rows(L)
    h = np.zeros((Mp, D), np.float32)
    h[:L] = W["embed"][np.asarray(ids)]
    xq, xs, _ = O.rmsnorm_quant(h, W["layers.0.input_layernorm"], eps, Mp)
    for i in range(a.num_hidden_layers):
        p = f"layers.{i}."
        wq, ws = _decoded(packed, [p + n for n in ATTN], fmt)
        y = O.epilogue(O.gemm_i32(xq, wq), xs, ws, 1)
        q, k, v = O.qkv_norm(y, W[p + "q_norm"], W[p + "k_norm"], eps, L, hq, hk, d, full=full, inv_freq=inv_freq, pos0=0)
        o = np.zeros((Mp, hq * d), np.float32)
        o[:L] = O.bf16_round(_attention(q, k, v, d ** -0.5).astype(np.float32))
        xq, xs = O.act_quant(o, Mp)
        wq, ws = _decoded(packed, [p + "self_attn.o_proj"], fmt)
        h = O.epilogue(O.gemm_i32(xq, wq), xs, ws, 2, res=h)
        nn = W[f"layers.{i + 1}.input_layernorm"] if i + 1 < a.num_hidden_layers else W["norm"]
        if a.num_experts:
            xq, xs, xn = O.rmsnorm_quant(h, W[p + "post_attention_layernorm"], eps, Mp)
            logits = O.bf16_round((xn[:L].astype(np.float64) @ W[p + "gate"].astype(np.float64).T).astype(np.float32))
            inds, scores = O.softmax_topk(logits, a.num_experts_per_tok)
            scores = O.bf16_round(scores)
            y = np.zeros((L, a.num_experts_per_tok, D), np.float32)
            for e in np.unique(inds):
                t, j = np.nonzero(inds == e)
                gq, gs = _decoded(packed, [p + f"experts.gate_proj.{e}", p + f"experts.up_proj.{e}"], fmt)
                act = O.epilogue(O.gemm_i32(xq[t], gq[perm]), xs[t], gs[perm], 3)
                aq, as_ = O.act_quant(act, len(t))
                dq, ds = _decoded(packed, [p + f"experts.down_proj.{e}"], fmt)
                y[t, j] = O.epilogue(O.gemm_i32(aq, dq), as_, ds, 1)
            k_ = a.num_experts_per_tok
            h = O.moe_combine(y.reshape(L * k_, D), np.arange(L * k_), scores, h, L)
        else:
            xq, xs, _ = O.rmsnorm_quant(h, W[p + "post_attention_layernorm"], eps, Mp)
            wq, ws = _decoded(packed, [p + "mlp.gate_proj", p + "mlp.up_proj"], fmt)
            act = O.epilogue(O.gemm_i32(xq, wq[perm]), xs, ws[perm], 3)
            xq, xs = O.act_quant(act, Mp)
            wq, ws = _decoded(packed, [p + "mlp.down_proj"], fmt)
            h = O.epilogue(O.gemm_i32(xq, wq), xs, ws, 2, res=h)
        if trace is not None:
            trace[i] = h[:L].copy()
        xq, xs, xn = O.rmsnorm_quant(h, nn, eps, Mp)
    head = W.get("lm_head", W["embed"])
    return O.bf16_round((xn[:L].astype(np.float64) @ head.astype(np.float64).T).astype(np.float32))
