"""CPU checks of the whole-model restatement (oracle/model_oracle.py) and of the packed-weight file format:
the float mode against the Hugging Face implementations of the two architectures, the W4A8 mode against the float mode
on the dequantized weights, safetensors round trips and the MXFP4 scale view."""
import importlib
import os
import types

import numpy as np
import pytest
import torch

import helpers as H

model_oracle = importlib.import_module("model_oracle")


def _args(cfg, model_type):
    return types.SimpleNamespace(
        hidden_size=cfg.hidden_size, intermediate_size=cfg.intermediate_size, num_hidden_layers=cfg.num_hidden_layers,
        num_attention_heads=cfg.num_attention_heads, num_key_value_heads=cfg.num_key_value_heads,
        head_dim=getattr(cfg, "head_dim", None) or cfg.hidden_size // cfg.num_attention_heads,
        rms_norm_eps=cfg.rms_norm_eps, rope_theta=_theta(cfg), vocab_size=cfg.vocab_size,
        tie_word_embeddings=cfg.tie_word_embeddings, num_experts=getattr(cfg, "num_experts", 0),
        num_experts_per_tok=getattr(cfg, "num_experts_per_tok", 0), norm_topk_prob=False, model_type=model_type)


def _theta(cfg):
    if getattr(cfg, "rope_theta", None):
        return cfg.rope_theta
    return cfg.rope_parameters["rope_theta"]


def _hf(kind):
    tr = pytest.importorskip("transformers")
    torch.manual_seed(0)
    if kind == "qwen3":
        cfg = tr.Qwen3Config(hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4,
                             num_key_value_heads=2, head_dim=32, vocab_size=97, rms_norm_eps=1e-6, rope_theta=1e6,
                             tie_word_embeddings=True, max_position_embeddings=128, attention_bias=False)
        m = tr.Qwen3ForCausalLM(cfg)
    else:
        cfg = tr.OlmoeConfig(hidden_size=128, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                             num_key_value_heads=4, vocab_size=97, num_experts=8, num_experts_per_tok=2,
                             norm_topk_prob=False, rms_norm_eps=1e-5, rope_theta=1e4, tie_word_embeddings=False,
                             max_position_embeddings=128)
        m = tr.OlmoeForCausalLM(cfg)
    m = m.eval().float()
    with torch.no_grad():                      # non-trivial norm weights, larger linears: a sharper wiring check
        for n, p in m.named_parameters():
            if "norm" in n:
                p.copy_(1 + 0.2 * torch.randn_like(p))
            elif p.ndim >= 2 and "embed" not in n:
                p.mul_(3.0)
    return m, _args(cfg, kind)


@pytest.mark.parametrize("kind", ["qwen3", "olmoe"])
def test_float_mode_matches_hugging_face(kind):
    m, args = _hf(kind)
    ids = np.random.default_rng(1).integers(0, args.vocab_size, 11)
    with torch.no_grad():
        ref = m(torch.from_numpy(ids)[None]).logits[0].double().numpy()
    W = H.oracle_weights(m.state_dict(), args)
    got = model_oracle.forward_float(W, args, ids)
    assert H.rel_l2(got, ref) < 2e-5


@pytest.mark.parametrize("kind", ["qwen3", "olmoe"])
def test_w4a8_mode_is_the_float_function_up_to_quantization(kind, oracle):
    m, args = _hf(kind)
    ids = np.random.default_rng(2).integers(0, args.vocab_size, 9)
    W = H.oracle_weights(m.state_dict(), args)
    W = {k: oracle.bf16_round(v) for k, v in W.items()}
    packed, deq = H.oracle_pack(W, oracle)
    ref = model_oracle.forward_float({**W, **deq}, args, ids)
    got = model_oracle.forward_w4a8(W, packed, args, ids)
    # INT8 activations + bf16 roundings on a 2-layer model: a few percent; a wiring error gives O(1)
    assert H.rel_l2(got, ref) < 0.08


def test_packed_file_round_trip_and_shift_layout(tmp_path, scmx, oracle):
    io = importlib.import_module("mxfp4-int8-m5_b200.packed_io")
    rng = np.random.default_rng(3)
    packed = {}
    for name, (n, k) in {"layers.0.self_attn.q_proj": (8, 256), "layers.0.experts.gate_proj.3": (4, 128)}.items():
        packed[name] = oracle.quantize(H.llm_weights(rng, n, k).astype(np.float64))[:3]
    path = os.path.join(tmp_path, "sub", "pack.safetensors")
    io.save_packed(path, packed)
    back = io.load_packed(path)
    assert set(back) == set(packed)
    for k in packed:
        for a, b in zip(packed[k], back[k]):
            assert a.dtype == b.dtype and np.array_equal(a.reshape(-1), b.reshape(-1))
    # the byte-shift cache layout (one shift byte per 32-block) loads to the same 2-bit block codes
    from safetensors.numpy import save_file
    flat = {}
    for k, (c, b, s) in packed.items():
        shifts = ((b[..., None] >> (2 * np.arange(4, dtype=np.uint8))) & 3).reshape(b.shape[0], -1).astype(np.uint8)
        flat[k + ".codes"], flat[k + ".shifts"], flat[k + ".wscale"] = c, shifts, s
    p2 = os.path.join(tmp_path, "shifts.safetensors")
    save_file(flat, p2)
    back2 = io.load_packed(p2)
    for k in packed:
        for a, b in zip(packed[k], back2[k]):
            assert np.array_equal(np.asarray(a).reshape(-1), np.asarray(b).reshape(-1))


def test_mxfp4_scale_view_decodes_to_the_same_weights(scmx, oracle):
    io = importlib.import_module("mxfp4-int8-m5_b200.packed_io")
    rng = np.random.default_rng(4)
    n, k = 16, 256
    codes, bc, ws = oracle.quantize(H.llm_weights(rng, n, k).astype(np.float64))[:3]
    scales = io.mxfp4_scales(bc, ws, k)
    assert scales.dtype == np.uint8 and scales.shape == (n, k // 32) and scales.flags.c_contiguous
    e2m1 = np.array([0, 0.5, 1, 1.5, 2, 3, 4, 6])
    nib = (codes.reshape(n, k // 8)[:, :, None] >> (4 * np.arange(8, dtype=np.uint32))) & 15
    nib = nib.reshape(n, k)
    val = np.where(nib & 8, -1.0, 1.0) * e2m1[nib & 7] * np.exp2(scales.astype(np.float64) - 127).repeat(32, axis=1)
    want = oracle.decode(codes, bc, n, k).astype(np.float64) * ws[:, None].astype(np.float64)
    assert np.array_equal(val, want)
    with pytest.raises(ValueError):
        io.mxfp4_scales(bc, ws * 1.5, k)
