"""The W4A8 part of a dense decoder stack as one chained call, the torch counterpart of the `post` / `pre` halves the
reference builds in FusedQwen3._block_fns (e2e/fused_qwen3.py:161-173): per layer
    rmsnorm_quant -> q|k|v GEMM (EPI 1) ; act_quant(attention output) -> o GEMM (+ residual) -> rmsnorm_quant ->
    gate|up GEMM (SwiGLU, rows interleaved) -> act_quant -> down GEMM (+ residual).
Attention itself (RoPE, KV cache, SDPA) is outside the W4A8 path; the caller supplies its output.

Every GEMM reads an INT8 operand decoded from the packed 4-bit codes just before it.  The decode of GEMM g+1 runs on a
side stream while GEMM g occupies the tensor cores (the reference overlaps the same two kernels through its `deps`
arguments, e2e/sc_kernels.py:18-20); two rotating scratch buffers stay resident in L2."""
import torch

from . import sc_kernels as S

GROUPS = ("qkv", "o", "gu", "down")


class DenseStack:
    def __init__(self, layers, M, hidden, eps=1e-6, overlap=True):
        """layers: list of {group: (codes, bcodes, wscale, N, K)} with gate|up rows already interleaved
        (sc_kernels.interleave_gate_up); M: rows (a multiple of 128); hidden: model width."""
        assert M % S.TM == 0
        self.layers, self.M, self.hidden, self.eps, self.overlap = layers, M, hidden, eps, overlap
        dev = layers[0]["qkv"][0].device
        big = max(n * k for lw in layers for (_, _, _, n, k) in lw.values())
        self.bufs = [torch.empty(big, dtype=torch.int8, device=dev) for _ in range(2)]
        self.nw = torch.ones(hidden, dtype=torch.bfloat16, device=dev)
        self.side = torch.cuda.Stream(device=dev) if overlap else None
        self.launches_per_layer = 12

    def packed_bytes(self):
        return sum(c.numel() * 4 + b.numel() + s.numel() * 4 for lw in self.layers for (c, b, s, _, _) in lw.values())

    def step(self, h, o, events=None):
        """h bf16 [M, hidden] residual stream, o bf16 [M, hidden] attention output used by every layer (a stand-in when
        benchmarking).  Returns the final residual stream.  `events`, when a list, receives (start, end, ops) CUDA-event
        triples around every GEMM launch."""
        M = self.M
        seq = [lw[g] for lw in self.layers for g in GROUPS]
        n = len(seq)
        main = torch.cuda.current_stream()
        ready, done = [None] * n, [None] * n

        def decode(g):
            codes, bc, _, N, K = seq[g]
            buf = self.bufs[g % 2][:N * K].view(N, K)
            if not self.overlap:
                S.unpack_i8(codes, bc, N, K, out=buf)
                return
            with torch.cuda.stream(self.side):
                if g >= 2:
                    self.side.wait_event(done[g - 2])        # the GEMM that last read this buffer
                S.unpack_i8(codes, bc, N, K, out=buf)
                ready[g] = torch.cuda.Event()
                ready[g].record(self.side)

        def gemm(g, xq, xs, epi, res=None):
            _, _, ws, N, K = seq[g]
            if g + 1 < n and self.overlap:
                decode(g + 1)                                # overlaps with this GEMM
            if self.overlap:
                main.wait_event(ready[g])
            else:
                decode(g)
            wq = self.bufs[g % 2][:N * K].view(N, K)
            if events is not None:
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
            y = S.mm_epi(xq, wq, xs, ws, epi, res=res)
            if events is not None:
                e1.record()
                events.append((e0, e1, 2 * xq.shape[0] * N * K))
            if self.overlap:
                done[g] = torch.cuda.Event()
                done[g].record(main)
            return y

        if self.overlap:
            self.side.wait_stream(main)
            decode(0)
        g = 0
        for _ in self.layers:
            xq, xs = S.rmsnorm_quant(h, self.nw, self.eps, M)
            gemm(g, xq, xs, 1)                               # q|k|v (consumed by attention, outside this path)
            oq, os_ = S.act_quant(o, M)
            h = gemm(g + 1, oq, os_, 2, res=h)
            xq, xs = S.rmsnorm_quant(h, self.nw, self.eps, M)
            act = gemm(g + 2, xq, xs, 3)
            aq, as_ = S.act_quant(act, M)
            h = gemm(g + 3, aq, as_, 2, res=h)
            g += 4
        if self.overlap:
            main.wait_stream(self.side)
        return h
