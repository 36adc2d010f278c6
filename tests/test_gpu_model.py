"""GPU checks of the callers around the W4A8 kernels: the q/k/v epilogue kernel against the oracle, and the fused prefill /
decode classes against the whole-model oracle, the unfused W4A8Linear model and each other."""
import copy
import importlib
import os

import numpy as np
import pytest
import torch

import helpers as H

pytestmark = pytest.mark.gpu
model_oracle = importlib.import_module("model_oracle")


def _mod(name):
    return importlib.import_module("mxfp4-int8-m5_b200." + name)


# ---- q/k/v epilogue kernel ---------------------------------------------------------------------------------------------

@pytest.mark.parametrize("full", [False, True])
@pytest.mark.parametrize("from_acc", [False, True])
@pytest.mark.parametrize("rope", [False, True])
def test_qkv_norm_matches_oracle(scmx, oracle, full, from_acc, rope):
    S = _mod("sc_kernels")
    HM = _mod("host_model")
    rng = np.random.default_rng(5)
    L, hq, hk, d = 37, 4, (4 if full else 2), 64
    ntot = (hq + 2 * hk) * d
    qn = oracle.bf16_round(1 + 0.2 * rng.standard_normal(hq * d if full else d).astype(np.float32))
    kn = oracle.bf16_round(1 + 0.2 * rng.standard_normal(hk * d if full else d).astype(np.float32))
    eps, off = 1e-6, 5
    inv = oracle.rope_inv_freq(d, 1e4) if rope else None
    if from_acc:
        acc = rng.integers(-200000, 200000, (L, ntot)).astype(np.int32)
        xs = (rng.random(L).astype(np.float32) + 0.5) * 1e-3
        ws = (rng.random(ntot).astype(np.float32) + 0.5) * 1e-2
        want = oracle.qkv_epilogue_headnorm(acc, xs, ws, qn, kn, eps, L, hq, hk, d, full=full, inv_freq=inv, pos0=off)
        src, cxs, cws = H.cuda(acc), H.cuda(xs), H.cuda(ws)
    else:
        y = oracle.bf16_round(rng.standard_normal((L, ntot)).astype(np.float32) * 3)
        want = oracle.qkv_norm(y, qn, kn, eps, L, hq, hk, d, full=full, inv_freq=inv, pos0=off)
        src, cxs, cws = H.to_bf16_cuda(y), None, None
    cache = HM.KVCache(hk, d, 64)
    cache.k.fill_(7.0), cache.v.fill_(7.0)
    cache.offset = off
    q, k, v = S._qkv_norm(src, cxs, cws, H.to_bf16_cuda(qn), H.to_bf16_cuda(kn), eps, L, hq, hk, d, full,
                          (H.cuda(inv), off) if rope else None, cache)
    torch.cuda.synchronize()
    assert k.shape == (hk, off + L, d)
    for got, ref in ((q, want[0]), (k[:, off:], want[1]), (v[:, off:], want[2])):
        assert np.array_equal(H.bf16_np(got), ref)
    # rows outside [offset, offset + L) of the cache are untouched
    assert bool((cache.k[:, :off] == 7).all()) and bool((cache.k[:, off + L:] == 7).all())
    assert bool((cache.v[:, :off] == 7).all()) and bool((cache.v[:, off + L:] == 7).all())
    if rope:       # the precomputed cos / sin table gives the same bits; positions past its end fall back to evaluation
        for rows in (64, off + 10):
            tab = S.rope_table(H.cuda(inv), rows)
            c3 = HM.KVCache(hk, d, 64)
            c3.offset = off
            q3, k3, v3 = S._qkv_norm(src, cxs, cws, H.to_bf16_cuda(qn), H.to_bf16_cuda(kn), eps, L, hq, hk, d, full,
                                     (H.cuda(inv), off, tab), c3)
            assert torch.equal(q3, q) and torch.equal(k3[:, off:], k[:, off:])
    # without a cache the outputs are fresh [h, L, d] tensors with the same values
    q2, k2, v2 = S._qkv_norm(src, cxs, cws, H.to_bf16_cuda(qn), H.to_bf16_cuda(kn), eps, L, hq, hk, d, full,
                             (H.cuda(inv), off) if rope else None, None)
    assert torch.equal(q2, q) and torch.equal(k2, k[:, off:]) and torch.equal(v2, v[:, off:])


def test_qkv_norm_device_side_position(scmx, oracle):
    S = _mod("sc_kernels")
    HM = _mod("host_model")
    rng = np.random.default_rng(6)
    hq, hk, d = 4, 2, 128
    y = H.to_bf16_cuda(oracle.bf16_round(rng.standard_normal((1, (hq + 2 * hk) * d)).astype(np.float32)))
    qn = kn = torch.ones(d, dtype=torch.bfloat16, device="cuda")
    inv = S.rope_inv_freq(d, 1e6)
    a, b = HM.KVCache(hk, d, 16), HM.KVCache(hk, d, 16)
    for c in (a, b):
        c.k.zero_(), c.v.zero_()
    a.offset = 9
    qa, _, _ = S.qkv_headnorm_y(y, qn, kn, 1e-6, 1, hq, hk, d, rope=(inv, 9), cache=a)
    step = torch.tensor([9], dtype=torch.int32, device="cuda")
    qb, _, _ = S.qkv_headnorm_y(y, qn, kn, 1e-6, 1, hq, hk, d, rope=(inv, 0), cache=b, pos_dev=step)
    assert torch.equal(qa, qb) and torch.equal(a.k, b.k) and torch.equal(a.v, b.v)
    # a device-side step beyond the cache drops the k / v rows instead of writing out of bounds
    step.fill_(16)
    before = b.k.clone()
    S.qkv_headnorm_y(y, qn, kn, 1e-6, 1, hq, hk, d, rope=(inv, 0), cache=b, pos_dev=step)
    torch.cuda.synchronize()
    assert torch.equal(before, b.k)


@pytest.mark.parametrize("hq,hk,d", [(4, 4, 64), (16, 8, 128), (8, 2, 128)])
@pytest.mark.parametrize("T", [1, 17, 600, 2049])
def test_decode_attention_kernel(scmx, hq, hk, d, T):
    S, HM = _mod("sc_kernels"), _mod("host_model")
    g = torch.Generator(device="cuda").manual_seed(T + d)
    cap = 2304
    c = HM.KVCache(hk, d, cap)
    c.k.copy_(torch.randn(c.k.shape, generator=g, device="cuda") * 1.5)
    c.v.copy_(torch.randn(c.v.shape, generator=g, device="cuda"))
    q = (torch.randn((hq, 1, d), generator=g, device="cuda") * 1.5).to(torch.bfloat16)
    att = S.DecodeAttention(hq, hk, d)
    want = HM.sdpa_f64(q, c.k[:, :T], c.v[:, :T], d ** -0.5, False).float()
    got = att(q, c, d ** -0.5, n_pos=T).float()
    assert H.rel_l2(got.cpu().numpy(), want.cpu().numpy()) < 4e-3          # one bf16 rounding of a float32 result
    pos = torch.tensor([T - 1], dtype=torch.int32, device="cuda")
    again = att(q, c, d ** -0.5, pos_dev=pos).float()                       # device-side length, second use of the scratch
    assert torch.equal(got, again)
    assert int(att.counters.abs().sum()) == 0


# ---- whole models ------------------------------------------------------------------------------------------------------

def _tiny(kind):
    HM = _mod("host_model")
    if kind == "qwen3":
        a = HM.ModelArgs(256, 512, 2, 4, 2, 64, 1e-6, 1e6, 512, True)
    else:
        a = HM.ModelArgs(256, 128, 2, 4, 4, 64, 1e-5, 1e4, 512, False, 8, 2, False, "olmoe")
    model = HM.CausalLM(a).init_random(seed=11, scale=0.05).cuda()
    return model, a


def _fused(kind, model, packed=None, **kw):
    if kind == "qwen3":
        FQ = _mod("fused_qwen3")
        packed = packed if packed is not None else FQ.pack_model(model)
        return FQ.FusedQwen3(model, packed, **kw), packed
    FO = _mod("fused_olmoe")
    packed = packed if packed is not None else FO.pack_olmoe(model)
    return FO.FusedOlmoe(model, packed, **kw), packed


def _ids(n, vocab, seed):
    return torch.from_numpy(np.random.default_rng(seed).integers(0, vocab, n)).cuda()[None]


@pytest.mark.parametrize("kind", ["qwen3", "olmoe"])
def test_fused_prefill_matches_model_oracle(scmx, oracle, kind):
    model, a = _tiny(kind)
    W = H.oracle_weights(model.state_dict(), a)
    fused, packed = _fused(kind, model)
    ids = _ids(150, a.vocab_size, 12)                 # pads to 256 rows
    want = model_oracle.forward_w4a8(W, packed, a, ids[0].cpu().numpy())
    # with attention evaluated in float64 (one rounding at its output, as in the oracle) every step of the chain is
    # reproduced bit for bit, up to a float64 summation-order tie in the attention output
    fused.sdpa = _mod("host_model").sdpa_f64
    exact = H.bf16_np(fused(ids))[0]
    assert H.rel_l2(exact, want) < 1e-4
    assert (exact != want).mean() < 1e-3
    # torch's bf16 attention kernel differs in the last bit of some outputs; the INT8 steps that follow amplify that
    fused.sdpa = _mod("host_model").sdpa
    got = H.bf16_np(fused(ids))[0]
    assert H.rel_l2(got, want) < 6e-2
    assert (got.argmax(-1) == want.argmax(-1)).mean() > 0.9


def test_fused_qwen3_variants_agree(scmx):
    FQ = _mod("fused_qwen3")
    model, a = _tiny("qwen3")
    packed = FQ.pack_model(model)
    ids = _ids(200, a.vocab_size, 13)
    outs = {}
    for name, kw in dict(ring=dict(overlap=True), serial=dict(overlap=False), resident=dict(resident=True),
                         row=dict(epilogue="row"), torch_rope=dict(fuse_rope=False)).items():
        f = FQ.FusedQwen3(copy.deepcopy(model), packed, **kw)
        outs[name] = f(ids)
    torch.cuda.synchronize()
    for name in ("serial", "resident", "row", "torch_rope"):
        # same kernels in another schedule / the row-kernel forms of the same epilogues: identical bits
        assert torch.equal(outs["ring"], outs[name]), name


@pytest.mark.parametrize("kind", ["qwen3"])
def test_fused_equals_unfused_w4a8_linear_model(scmx, kind):
    W4 = _mod("w4a8")
    model, a = _tiny(kind)
    unfused = copy.deepcopy(model)
    fused, packed = _fused(kind, model)
    W4.apply_w4a8(unfused, packed)
    ids = _ids(130, a.vocab_size, 14)
    with torch.no_grad():
        ref = unfused(ids).float().cpu().numpy()[0]
    got = H.bf16_np(fused(ids))[0]
    # the unfused model rounds gate and up to bf16 separately and uses torch's silu: not bit-equal, same function
    assert H.rel_l2(got, ref) < 5e-2


@pytest.mark.parametrize("kind", ["qwen3", "olmoe"])
def test_decode_steps_match_prefill(scmx, kind):
    DEC, HM = _mod("decode"), _mod("host_model")
    model, a = _tiny(kind)
    fused, packed = _fused(kind, model)
    cls = DEC.DecodeQwen3 if kind == "qwen3" else DEC.DecodeOlmoe
    ids = _ids(40, a.vocab_size, 15)
    n0 = 36
    # attention in float64 on both sides: what remains are the GEMVs against the GEMMs (exact integers both) and the row
    # kernels at M = 1 against M = 128 k, so a decode step reproduces the prefill's logits
    fused.sdpa = HM.sdpa_f64
    dec = cls(fused, attention="torch")
    cache = fused.make_cache(64)
    fused(ids[:, :n0], cache)
    full = fused(ids)                                   # logits of every prefix from one prefill
    for t in range(n0, 40):
        step = dec.step(ids[:, t:t + 1], cache)
        assert cache[0].offset == t + 1
        got, want = H.bf16_np(step[0, 0]), H.bf16_np(full[0, t])
        assert H.rel_l2(got, want) < 1e-3
        assert got.argmax() == want.argmax()
    # default attention (torch's kernel in the prefill, the library's decode kernel in the step): last-bit differences
    # of the attention outputs, amplified by the INT8 steps of a small random model
    fused.sdpa = HM.sdpa
    dec = cls(fused)
    cache = fused.make_cache(64)
    fused(ids[:, :n0], cache)
    full = fused(ids)
    step = dec.step(ids[:, n0:n0 + 1], cache)
    assert H.rel_l2(H.bf16_np(step[0, 0]), H.bf16_np(full[0, n0])) < 8e-2


def test_prefill_into_offset_cache(scmx):
    model, a = _tiny("qwen3")
    fused, _ = _fused("qwen3", model)
    ids = _ids(96, a.vocab_size, 16)
    whole = fused(ids)
    cache = fused.make_cache(128)
    fused(ids[:, :50], cache)
    second = fused(ids[:, 50:], cache)
    assert H.rel_l2(H.bf16_np(second[0]), H.bf16_np(whole[0, 50:])) < 8e-2


def test_pack_cache_file_round_trip(scmx, tmp_path):
    FQ = _mod("fused_qwen3")
    model, a = _tiny("qwen3")
    path = os.path.join(tmp_path, "tiny-scmxfp4.safetensors")
    packed = FQ.pack_model(model, path)
    assert os.path.exists(path)
    again = FQ.pack_model(model, path)                 # second call reads the file
    loaded = FQ.load_packed(path, a.num_hidden_layers)
    for k in packed:
        for x, y, z in zip(packed[k], again[k], loaded[k]):
            assert np.array_equal(np.asarray(x).reshape(-1), np.asarray(y).reshape(-1))
            assert np.array_equal(np.asarray(x).reshape(-1), np.asarray(z).reshape(-1))
    ids = _ids(64, a.vocab_size, 17)
    a1 = FQ.FusedQwen3(copy.deepcopy(model), packed)(ids)
    a2 = FQ.FusedQwen3(copy.deepcopy(model), loaded)(ids)
    a3 = FQ.FusedQwen3(copy.deepcopy(model), FQ.pack_model(model, on_device=True))(ids)
    assert torch.equal(a1, a2) and torch.equal(a1, a3)


@pytest.mark.parametrize("kind", ["qwen3", "olmoe"])
def test_graph_generate_equals_eager_steps(scmx, kind):
    DEC = _mod("decode")
    model, a = _tiny(kind)
    fused, _ = _fused(kind, model)
    dec = (DEC.DecodeQwen3 if kind == "qwen3" else DEC.DecodeOlmoe)(fused)
    assert dec.attention == "kernel"
    ids = _ids(24, a.vocab_size, 18)
    n = 12

    def prompt():
        cache = fused.make_cache(64)
        logits = fused(ids, cache)
        return cache, logits[:, -1].argmax(-1, keepdim=True)

    cache, tok = prompt()
    eager = []
    for _ in range(n):
        tok = dec.step(tok, cache)[:, -1].argmax(-1, keepdim=True)
        eager.append(int(tok))
    cache2, tok2 = prompt()
    got = dec.generate(tok2, cache2, n).tolist()
    assert got == eager and cache2[0].offset == 24 + n
    assert torch.equal(cache[0].k[:, :24 + n], cache2[0].k[:, :24 + n])
    # a second run on the same cache object reuses the captured graph from a new start position
    for c in cache2:
        c.offset = 24
    assert dec.generate(tok2, cache2, n).tolist() == eager
    # the kernel attention and torch's agree to bf16 accuracy on a step
    dec_t = (DEC.DecodeQwen3 if kind == "qwen3" else DEC.DecodeOlmoe)(fused, attention="torch")
    c1, t1 = prompt()
    c2, _ = prompt()
    l1, l2 = dec.step(t1, c1), dec_t.step(t1, c2)
    assert H.rel_l2(H.bf16_np(l1[0, 0]), H.bf16_np(l2[0, 0])) < 8e-2


def test_persistent_decode_kernel_equals_kernel_chain(scmx):
    """All layers of a step in one cooperative kernel against the chain of stand-alone kernels: same logits, bit for bit,
    same cache contents, eagerly and replayed from a CUDA graph."""
    HM, FQ, DEC = _mod("host_model"), _mod("fused_qwen3"), _mod("decode")
    a = HM.ModelArgs(1024, 3072, 2, 8, 4, 128, 1e-6, 1e6, 512, True)
    model = HM.CausalLM(a).init_random(seed=21, scale=0.05).cuda()
    fused = FQ.FusedQwen3(model, FQ.pack_model(model, on_device=True))
    chain = DEC.DecodeQwen3(fused, persistent=False)
    mk = DEC.DecodeQwen3(fused, persistent=True)
    assert mk.persistent and not chain.persistent
    ids = _ids(150, a.vocab_size, 22)
    n = 6

    def prompt(L):
        cache = fused.make_cache(256)
        return cache, fused(ids[:, :L], cache)[:, -1].argmax(-1, keepdim=True)

    for L in (5, 70, 150):                                # 1, 2 and 3 attention splits in use
        c1, t1 = prompt(L)
        c2, t2 = prompt(L)
        for _ in range(n):
            l1, l2 = chain.step(t1, c1), mk.step(t2, c2)
            assert torch.equal(l1, l2)
            t1 = l1[:, -1].argmax(-1, keepdim=True)
            t2 = l2[:, -1].argmax(-1, keepdim=True)
        mk.check_status()
        for x, y in zip(c1, c2):
            assert x.offset == y.offset == L + n
            assert torch.equal(x.k[:, :L + n], y.k[:, :L + n]) and torch.equal(x.v[:, :L + n], y.v[:, :L + n])
    c1, t1 = prompt(40)
    c2, t2 = prompt(40)
    assert chain.generate(t1, c1, n).tolist() == mk.generate(t2, c2, n).tolist()
    mk.check_status()
    assert torch.equal(c1[1].k[:, :40 + n], c2[1].k[:, :40 + n])


def test_fused_qwen3_rotated_inputs_path(scmx):
    """rot=True / "down" route the INT8 quantization of the GEMM inputs through rot_quant (for packs made in the rotated
    basis); with ordinary packs the outputs are simply different, finite numbers - this checks the wiring only."""
    FQ, S = _mod("fused_qwen3"), _mod("sc_kernels")
    model, a = _tiny("qwen3")
    packed = FQ.pack_model(model)
    ids = _ids(70, a.vocab_size, 19)
    base = FQ.FusedQwen3(copy.deepcopy(model), packed)(ids)
    for rot in (True, "down"):
        f = FQ.FusedQwen3(copy.deepcopy(model), packed, rot=rot)
        x = torch.randn((128, a.intermediate_size), device="cuda").to(torch.bfloat16)
        q1, s1 = f.act_q(x, 128, down=True)
        q2, s2 = S.rot_quant(x, S.rot_signs(a.intermediate_size), 128)
        assert torch.equal(q1, q2) and torch.equal(s1, s2)
        q3, _ = f.act_q(x, 128)
        assert torch.equal(q3, q2) == (rot is True)
        out = f(ids)
        assert torch.isfinite(out.float()).all() and not torch.equal(out, base)
