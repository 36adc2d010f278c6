"""One mixture-of-experts half-block of the W4A8 path as a chained call, the torch counterpart of the expert part of
FusedOlmoe's `post` (e2e/fused_olmoe.py:211-245): RMSNorm + INT8 -> router softmax/top-k -> counting sort -> row gather ->
gate|up grouped GEMM with SwiGLU -> act_quant -> down grouped GEMM -> weighted bf16 combine + residual."""
import torch

from . import sc_kernels as S
from . import sc_moe as M_


class MoeBlock:
    def __init__(self, gu, dn, n_experts, topk, D, F, eps=1e-5, two_pass=False):
        """gu = (codes [E, 2F*D/8], bcodes [E, 2F, D/128], wscale [E, 2F]) with gate|up rows interleaved;
        dn = (codes [E, D*F/8], bcodes [E, D, F/128], wscale [E, D]).  two_pass: keep the experts decoded to INT8
        (moe_mm_i8) instead of decoding per call (moe_mm)."""
        self.gu, self.dn, self.E, self.k, self.D, self.F, self.eps = gu, dn, n_experts, topk, D, F, eps
        self.nw = torch.ones(D, dtype=torch.bfloat16, device=gu[0].device)
        self.two_pass = two_pass
        if two_pass:
            self.gu8 = M_.unpack_experts(gu[0], gu[1], 2 * F, D)
            self.dn8 = M_.unpack_experts(dn[0], dn[1], D, F)

    def experts(self, xq_s, xs_s, R, off, ts, mt):
        """Sorted INT8 rows [R + 128, D] -> bf16 expert outputs [R, D]."""
        D, F = self.D, self.F
        if self.two_pass:
            act = M_.moe_mm_i8(xq_s, R, self.gu8, self.gu[2], off, ts, mt, 2 * F, 3, xs_s)
        else:
            act = M_.moe_mm(xq_s, R, *self.gu, off, ts, mt, 2 * F, 3, xs_s)
        xq2, xs2 = S.act_quant(act, R + M_.TM)
        if self.two_pass:
            return M_.moe_mm_i8(xq2, R, self.dn8, self.dn[2], off, ts, mt, D, 1, xs2)
        return M_.moe_mm(xq2, R, *self.dn, off, ts, mt, D, 1, xs2)

    def step(self, h, logits):
        """h bf16 [L, D] (L a multiple of 128), router logits f32 [L, E] -> new residual stream bf16 [L, D]."""
        L = h.shape[0]
        R = L * self.k
        xq, xs = S.rmsnorm_quant(h, self.nw, self.eps, L)
        inds, scores = M_.router_topk(logits, self.k)
        pos, tok, _, off, ts, mt = M_.route_sort(inds, self.E, M_.TM)
        xq_s, xs_s = M_.gather_rows(xq, xs, tok, R)
        yd = self.experts(xq_s, xs_s, R, off, ts, mt)
        hout, _, _ = M_.moe_combine(yd, pos, scores, h, self.nw, self.eps, L, quant=False)
        return hout
