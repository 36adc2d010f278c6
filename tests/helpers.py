"""Shared helpers of the test-suite: bf16 <-> NumPy conversion, seeded inputs in the reference's recipes."""
import hashlib

import numpy as np
import torch


def sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()[:16]


def to_bf16_cuda(x_f32):
    """float32 NumPy array holding bf16-representable values -> CUDA bfloat16 tensor."""
    return torch.from_numpy(np.ascontiguousarray(x_f32, np.float32)).cuda().to(torch.bfloat16)


def bf16_np(t):
    """bfloat16 tensor -> float32 NumPy array."""
    return t.detach().float().cpu().numpy()


def cuda(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def llm_weights(rng, n, k, sigma=0.3):
    """w = N(0,1) * 0.02 * lognormal(0, sigma) per column (sim/make_testcase.py:48-50)."""
    return (rng.standard_normal((n, k)) * 0.02 * rng.lognormal(0, sigma, (1, k))).astype(np.float32)


def llm_acts(rng, m, k, oracle, outliers=8):
    """x = N(0,1) * lognormal(0, 0.5) per column with a few x20 outlier channels, rounded to bf16
    (sim/make_testcase.py:51-53)."""
    x = rng.standard_normal((m, k)) * rng.lognormal(0, 0.5, (1, k))
    x[:, rng.choice(k, outliers, replace=False)] *= 20
    return oracle.bf16_round(x.astype(np.float32))


def rel_l2(a, b):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return float(np.sqrt(((a - b) ** 2).sum() / max((b ** 2).sum(), 1e-300)))


# ---- whole-model helpers ----------------------------------------------------------------------------------------------

def oracle_weights(sd, args, f=lambda t: t.detach().float().cpu().numpy()):
    """Hugging Face style state dict (tensors) -> the flat weight dict of oracle/model_oracle.py.  Expert weights may be
    stored per expert (model.layers.i.mlp.experts.e.gate_proj.weight), stacked as switch_mlp.<proj>.weight [E, out, in],
    or fused as experts.gate_up_proj [E, 2F, D] / experts.down_proj [E, D, F]."""
    W = {"embed": f(sd["model.embed_tokens.weight"]), "norm": f(sd["model.norm.weight"])}
    if "lm_head.weight" in sd and not args.tie_word_embeddings:
        W["lm_head"] = f(sd["lm_head.weight"])
    Fi = args.intermediate_size
    for i in range(args.num_hidden_layers):
        p, q = f"model.layers.{i}.", f"layers.{i}."
        for n in ("input_layernorm", "post_attention_layernorm"):
            W[q + n] = f(sd[p + n + ".weight"])
        W[q + "q_norm"], W[q + "k_norm"] = f(sd[p + "self_attn.q_norm.weight"]), f(sd[p + "self_attn.k_norm.weight"])
        for n in ("q_proj", "k_proj", "v_proj", "o_proj"):
            if p + f"self_attn.{n}.weight" in sd:
                W[q + f"self_attn.{n}"] = f(sd[p + f"self_attn.{n}.weight"])
        if not getattr(args, "num_experts", 0):
            for n in ("gate_proj", "up_proj", "down_proj"):
                if p + f"mlp.{n}.weight" in sd:
                    W[q + f"mlp.{n}"] = f(sd[p + f"mlp.{n}.weight"])
            continue
        W[q + "gate"] = f(sd[p + "mlp.gate.weight"])
        for e in range(args.num_experts):
            if p + "mlp.experts.gate_up_proj" in sd:
                gu = f(sd[p + "mlp.experts.gate_up_proj"][e])
                parts = {"gate_proj": gu[:Fi], "up_proj": gu[Fi:], "down_proj": f(sd[p + "mlp.experts.down_proj"][e])}
            elif p + "mlp.switch_mlp.gate_proj.weight" in sd:
                parts = {n: f(sd[p + f"mlp.switch_mlp.{n}.weight"][e]) for n in ("gate_proj", "up_proj", "down_proj")}
            elif p + f"mlp.experts.{e}.gate_proj.weight" in sd:
                parts = {n: f(sd[p + f"mlp.experts.{e}.{n}.weight"]) for n in ("gate_proj", "up_proj", "down_proj")}
            else:
                break
            for n, w in parts.items():
                W[q + f"experts.{n}.{e}"] = w
    return W


def oracle_pack(W, oracle, names=None):
    """SC-MXFP4 of every linear of an oracle weight dict with the CPU quantizer -> ({name: (codes, bcodes, wscale)},
    dict of dequantized weights under the same names)."""
    packed, deq = {}, {}
    for k, w in W.items():
        if w.ndim != 2 or k in ("embed", "lm_head") or k.endswith(".gate"):
            continue
        if names is not None and k not in names:
            continue
        codes, bc, ws = oracle.quantize(w.astype(np.float64))[:3]
        packed[k] = (codes, bc, ws)
        deq[k] = oracle.decode(codes, bc, w.shape[0], w.shape[1]).astype(np.float32) * ws[:, None]
    return packed, deq
