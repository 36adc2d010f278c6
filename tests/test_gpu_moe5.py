"""GPU: the large-MoE stress configuration in small: block-16 format family (e2m1 codes, multipliers 1, 2, 4, 8) packed by the
device quantizer, Zipf-skewed routing (popular experts get most rows, some get none), grouped GEMMs gate|up (SwiGLU) and down
for 2 layers x 4 experts against the oracle's family quantizer and per-expert loop; both grouped forms (tiles expanded inside
the kernel, and decode-then-GEMM) and the gather GEMV of the decode step."""
import numpy as np
import pytest
import torch

from helpers import bf16_np, cuda

pytestmark = pytest.mark.gpu


def test_block16_family_grouped_gemm_under_skewed_routing(scmx, oracle):
    S, M_, F, G = scmx.sc_kernels, scmx.sc_moe, scmx.sc_format, scmx.sc_decode
    fmt = F.Format(block=16)
    ofmt = oracle.Format(block=16)
    rng = np.random.default_rng(5)
    E, D, Fd, tokens, k = 4, 512, 256, 300, 2
    S.set_format(fmt)
    try:
        for layer in range(2):
            gu_w = [(rng.standard_normal((2 * Fd, D)) * 0.02).astype(np.float32) for _ in range(E)]
            dn_w = [(rng.standard_normal((D, Fd)) * 0.02).astype(np.float32) for _ in range(E)]
            perm = S.interleave_gate_up(Fd)
            dev_gu = [F.family_quantize_device(cuda(w[perm]), fmt) for w in gu_w]
            dev_dn = [F.family_quantize_device(cuda(w), fmt) for w in dn_w]
            o_gu = [oracle.family_pack(w[perm], ofmt) for w in gu_w]
            o_dn = [oracle.family_pack(w, ofmt) for w in dn_w]
            for d_, o_ in zip(dev_gu + dev_dn, o_gu + o_dn):      # packed bits equal the oracle's
                assert np.array_equal(d_[0].cpu().numpy().view(np.uint32), o_[0]) and np.array_equal(d_[1].cpu().numpy(), o_[1])
                assert np.array_equal(d_[2].cpu().numpy(), o_[2]) and np.array_equal(d_[3].cpu().numpy(), o_[3])
            # Zipf(1.2) popularity over a permutation of the experts; the least popular expert gets no row at all
            pmf = np.arange(1, E + 1, dtype=np.float64) ** -1.2
            logits = rng.standard_normal((tokens, E)) + np.log(pmf / pmf.sum())[rng.permutation(E)][None, :]
            logits[:, int(np.argmin(logits.mean(0)))] = -30.0
            inds, scores = M_.router_topk(cuda(logits.astype(np.float32)), k)
            pos, tok, es, off, ts, mt = M_.route_sort(inds, E, 128)
            R = tokens * k
            off_n, tok_n = off.cpu().numpy(), tok.cpu().numpy()
            assert (np.diff(off_n) == 0).any() and np.diff(off_n).max() > R // E      # an empty expert and a popular one
            xq = rng.integers(-127, 128, (tokens, D)).astype(np.int8)
            xs = (np.abs(rng.standard_normal(tokens)) * 1e-2).astype(np.float32)
            xq_s = cuda(np.concatenate([xq[tok_n[:R]], np.zeros((128, D), np.int8)]))
            xs_s = cuda(xs[tok_n[:R]])
            cg, bg, sg = (torch.stack([d_[i] for d_ in dev_gu]) for i in range(3))
            cd, bd, sd = (torch.stack([d_[i] for d_ in dev_dn]) for i in range(3))
            want_acc = oracle.moe_mm(xq[tok_n[:R]], R, [o_[3] for o_ in o_gu], off_n, 0)
            want_act = oracle.moe_mm(xq[tok_n[:R]], R, [o_[3] for o_ in o_gu], off_n, 3, xs[tok_n[:R]], [o_[2] for o_ in o_gu])
            for fused in (True, False):
                M_.FUSED_UNPACK = fused
                acc = M_.moe_mm(xq_s, R, cg, bg, sg, off, ts, mt, 2 * Fd, 0)
                assert np.array_equal(acc.cpu().numpy(), want_acc), ("acc", fused)
                act = M_.moe_mm(xq_s, R, cg, bg, sg, off, ts, mt, 2 * Fd, 3, xs_s)
                bad = np.flatnonzero((bf16_np(act) != want_act).ravel())
                assert bad.size <= 2, ("swiglu", fused, bad.size)       # expf against a correctly rounded exp: one gate value
            M_.FUSED_UNPACK = True
            a_dev = bf16_np(act)
            xq2, xs2 = S.act_quant(act, R + 128)
            oq2, os2 = oracle.act_quant(a_dev)
            assert np.array_equal(xq2[:R].cpu().numpy(), oq2)
            yd = M_.moe_mm(xq2, R, cd, bd, sd, off, ts, mt, D, 1, xs2)
            assert np.array_equal(bf16_np(yd), oracle.moe_mm(oq2, R, [o_[3] for o_ in o_dn], off_n, 1, os2, [o_[2] for o_ in o_dn]))
            # decode step: the gather GEMV of one token over its two experts
            e1 = inds[0].to(torch.int32)
            y1 = G.gemv(cuda(xq[0]), cg, bg, cuda(xs[:1]), sg, 2 * Fd, 1, eidx=e1, xstride=0)
            for j, e in enumerate(e1.cpu().tolist()):
                assert np.array_equal(bf16_np(y1[j]), oracle.gemv(xq[0], xs[0], o_gu[e][3], o_gu[e][2], 1))
        torch.cuda.synchronize()
        scmx._lib.check_status()
    finally:
        M_.FUSED_UNPACK = True
        S.set_format(F.Format())
