"""One mixture-of-experts half-block of the W4A8 path as a chained call, the torch counterpart of the expert part of
FusedOlmoe's `post` (e2e/fused_olmoe.py:211-245): RMSNorm + INT8 -> router softmax/top-k -> counting sort -> row gather ->
gate|up grouped GEMM with SwiGLU -> act_quant -> down grouped GEMM -> weighted bf16 combine + residual."""
import torch

from . import sc_kernels as S
from . import sc_moe as M_


class MoeBlock:
    def __init__(self, gu, dn, n_experts, topk, D, F, eps=1e-5, two_pass=False, early_decode=True):
        """gu = (codes [E, 2F*D/8], bcodes [E, 2F, D/128], wscale [E, 2F]) with gate|up rows interleaved;
        dn = (codes [E, D*F/8], bcodes [E, D, F/128], wscale [E, D]).  two_pass: keep the experts decoded to INT8
        (moe_mm_i8) instead of decoding per call.  early_decode (default, when the INT8 copies of all experts fit in
        1 GiB): every step decodes all experts to INT8 on a side stream starting at the top of the step, under the
        RMSNorm / router / sort / gather kernels and the first grouped GEMM, and the GEMMs run on that (moe_mm_i8);
        otherwise moe_mm decodes groups of experts between its GEMM passes.  With fewer than FUSED_BELOW rows per expert on
        average (the reference's rule, e2e/fused_olmoe.py:205: two passes pay only when R // E >= 256) the grouped GEMM reads
        the packed weights directly and expands them inside its K loop (sc_moe.moe_mm -> scmx_moe_mm_w4): nothing is decoded
        to memory for a handful of rows per expert."""
        self.gu, self.dn, self.E, self.k, self.D, self.F, self.eps = gu, dn, n_experts, topk, D, F, eps
        dev = gu[0].device
        self.nw = torch.ones(D, dtype=torch.bfloat16, device=dev)
        self.two_pass = two_pass
        self.early = bool(early_decode and not two_pass and n_experts * 3 * F * D <= (1 << 30))
        if two_pass:
            self.gu8 = M_.unpack_experts(gu[0], gu[1], 2 * F, D)
            self.dn8 = M_.unpack_experts(dn[0], dn[1], D, F)
        elif self.early:
            self.gu8 = torch.empty((n_experts * 2 * F, D), dtype=torch.int8, device=dev)
            self.dn8 = torch.empty((n_experts * D, F), dtype=torch.int8, device=dev)
            self.side = torch.cuda.Stream(device=dev)

    # measured on B200 (64 experts, 2048 x 1024; half-block ms, packed-weight GEMMs / decode-then-GEMM): 128 rows per expert
    # 0.190 / 0.275, 256: 0.286 / 0.330, 384: 0.356 / 0.394, 448: 0.367 / 0.419, 512: 0.478 / 0.449 (past 512 rows an expert
    # needs a second super tile)
    FUSED_BELOW = 480

    def _fused(self, R):
        return (not self.two_pass) and M_.FUSED_UNPACK and R // self.E < self.FUSED_BELOW

    def _start_decode(self):
        """Both expert sets -> INT8 on the side stream; returns the events the two GEMMs wait for."""
        main = torch.cuda.current_stream()
        self.side.wait_stream(main)                           # the previous step's GEMMs no longer read the buffers
        E, D, F = self.E, self.D, self.F
        with torch.cuda.stream(self.side):
            S.unpack_i8(self.gu[0].reshape(-1), self.gu[1].reshape(E * 2 * F, -1), E * 2 * F, D, out=self.gu8)
            e_gu = torch.cuda.Event()
            e_gu.record(self.side)
            S.unpack_i8(self.dn[0].reshape(-1), self.dn[1].reshape(E * D, -1), E * D, F, out=self.dn8)
            e_dn = torch.cuda.Event()
            e_dn.record(self.side)
        return e_gu, e_dn

    def experts(self, xq_s, xs_s, R, off, ts, mt, decoded=None):
        """Sorted INT8 rows [R + 128, D] -> bf16 expert outputs [R, D]."""
        D, F = self.D, self.F
        main = torch.cuda.current_stream()
        fused = self._fused(R)
        if self.early and decoded is None and not fused:      # called on its own: decode now (still on the side stream)
            decoded = self._start_decode()
        if fused:
            act = M_.moe_mm(xq_s, R, *self.gu, off, ts, mt, 2 * F, 3, xs_s)
        elif self.two_pass or self.early:
            if decoded is not None:
                main.wait_event(decoded[0])
            act = M_.moe_mm_i8(xq_s, R, self.gu8, self.gu[2], off, ts, mt, 2 * F, 3, xs_s)
        else:
            act = M_.moe_mm(xq_s, R, *self.gu, off, ts, mt, 2 * F, 3, xs_s)
        xq2, xs2 = S.act_quant(act, R + M_.TM)
        if fused:
            return M_.moe_mm(xq2, R, *self.dn, off, ts, mt, D, 1, xs2)
        if self.two_pass or self.early:
            if decoded is not None:
                main.wait_event(decoded[1])
            return M_.moe_mm_i8(xq2, R, self.dn8, self.dn[2], off, ts, mt, D, 1, xs2)
        return M_.moe_mm(xq2, R, *self.dn, off, ts, mt, D, 1, xs2)

    def step(self, h, logits):
        """h bf16 [L, D] (L a multiple of 128), router logits f32 [L, E] -> new residual stream bf16 [L, D]."""
        L = h.shape[0]
        R = L * self.k
        decoded = self._start_decode() if (self.early and not self._fused(R)) else None
        # routing (top-k, counting sort) does not depend on the quantized rows: it runs beside RMSNorm + INT8 on a stream of its own
        main = torch.cuda.current_stream()
        if not hasattr(self, "route_stream"):
            self.route_stream = torch.cuda.Stream(device=h.device)
        self.route_stream.wait_stream(main)
        with torch.cuda.stream(self.route_stream):
            inds, scores = M_.router_topk(logits, self.k)
            pos, tok, _, off, ts, mt = M_.route_sort(inds, self.E, M_.TM)
        xq, xs = S.rmsnorm_quant(h, self.nw, self.eps, L)
        main.wait_stream(self.route_stream)
        xq_s, xs_s = M_.gather_rows(xq, xs, tok, R)
        yd = self.experts(xq_s, xs_s, R, off, ts, mt, decoded)
        hout, _, _ = M_.moe_combine(yd, pos, scores, h, self.nw, self.eps, L, quant=False)
        if decoded is not None:
            torch.cuda.current_stream().wait_stream(self.side)
        return hout
