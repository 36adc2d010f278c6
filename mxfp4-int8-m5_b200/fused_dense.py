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


class DecodeRing:
    """Schedules the 4-bit -> INT8 decode of a sequence of weights around the GEMMs that consume them: two rotating
    scratch buffers, the decode of weight g + 1 issued on a side stream just before GEMM g is launched, events in both
    directions (decoded -> GEMM may start; GEMM finished -> its buffer may be overwritten).  Capturable in a CUDA graph."""

    def __init__(self, max_elems, device, overlap=True):
        self.bufs = [torch.empty(max_elems, dtype=torch.int8, device=device) for _ in range(2)]
        self.overlap = overlap
        self.side = torch.cuda.Stream(device=device) if overlap else None

    def begin(self, seq):
        """seq: list of (codes, bcodes, wscale, N, K) in the order the GEMMs run."""
        self.seq, n = seq, len(seq)
        self.ready, self.done = [None] * n, [None] * n
        self.main = torch.cuda.current_stream()
        if self.overlap:
            self.side.wait_stream(self.main)
            self._decode(0)

    def _view(self, g):
        _, _, _, N, K = self.seq[g]
        return self.bufs[g % 2][:N * K].view(N, K)

    def _decode(self, g):
        codes, bc, _, N, K = self.seq[g]
        if not self.overlap:
            S.unpack_i8(codes, bc, N, K, out=self._view(g))
            return
        with torch.cuda.stream(self.side):
            if g >= 2:
                self.side.wait_event(self.done[g - 2])       # the GEMM that last read this buffer
            S.unpack_i8(codes, bc, N, K, out=self._view(g))
            self.ready[g] = torch.cuda.Event()
            self.ready[g].record(self.side)

    def weight(self, g):
        """INT8 operand of GEMM g; call right before launching it."""
        if self.overlap:
            if g + 1 < len(self.seq):
                self._decode(g + 1)                          # overlaps with GEMM g
            self.main.wait_event(self.ready[g])
        else:
            self._decode(g)
        return self._view(g)

    def released(self, g):
        """Call right after launching GEMM g."""
        if self.overlap:
            self.done[g] = torch.cuda.Event()
            self.done[g].record(self.main)

    def end(self):
        if self.overlap:
            self.main.wait_stream(self.side)


class DenseStack:
    def __init__(self, layers, M, hidden, eps=1e-6, overlap=True):
        """layers: list of {group: (codes, bcodes, wscale, N, K)} with gate|up rows already interleaved
        (sc_kernels.interleave_gate_up); M: rows (a multiple of 128); hidden: model width."""
        assert M % S.TM == 0
        self.layers, self.M, self.hidden, self.eps, self.overlap = layers, M, hidden, eps, overlap
        dev = layers[0]["qkv"][0].device
        big = max(n * k for lw in layers for (_, _, _, n, k) in lw.values())
        self.ring = DecodeRing(big, dev, overlap)
        self.nw = torch.ones(hidden, dtype=torch.bfloat16, device=dev)
        self.launches_per_layer = 12

    def packed_bytes(self):
        return sum(c.numel() * 4 + b.numel() + s.numel() * 4 for lw in self.layers for (c, b, s, _, _) in lw.values())

    def step(self, h, o, events=None):
        """h bf16 [M, hidden] residual stream, o bf16 [M, hidden] attention output used by every layer (a stand-in when
        benchmarking).  Returns the final residual stream.  `events`, when a list, receives (start, end, ops) CUDA-event
        triples around every GEMM launch."""
        M, ring = self.M, self.ring
        seq = [lw[g] for lw in self.layers for g in GROUPS]
        ring.begin(seq)

        def gemm(g, xq, xs, epi, res=None):
            _, _, ws, N, K = seq[g]
            wq = ring.weight(g)
            if events is not None:
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
            y = S.mm_epi(xq, wq, xs, ws, epi, res=res)
            if events is not None:
                e1.record()
                events.append((e0, e1, 2 * xq.shape[0] * N * K))
            ring.released(g)
            return y

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
        ring.end()
        return h
