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
    """Schedules the 4-bit -> INT8 decode of a sequence of weights around the GEMMs that consume them.  The sequence is cut into
    groups of `group` consecutive weights; two rotating sets of scratch buffers hold the current and the next group.  The decode
    of group j + 1 is issued on a side stream when group j is joined, events in both directions (group decoded -> its GEMMs may
    start; last GEMM of a group launched -> its buffers may be overwritten).  Capturable in a CUDA graph.

    group = 1 (the default) decodes weight g + 1 while GEMM g runs and joins the side stream before every GEMM: two buffers of
    one weight each, which stay in L2.  Larger groups join less often (group = 4: once per layer) but decode a whole layer in
    one burst into buffers that no longer fit L2; measured on the Qwen3-1.7B-shaped step at M = 2048: 4.39 ms with group 1,
    4.48 ms with 2, 4.57 ms with 4 (same GPU, same run)."""

    def __init__(self, max_elems, device, overlap=True, group=1):
        self.group, self.device = group, device
        self.sizes = [max_elems] * group if isinstance(max_elems, int) else list(max_elems)
        assert len(self.sizes) == group
        self.bufs = [[torch.empty(n, dtype=torch.int8, device=device) for n in self.sizes] for _ in range(2)]
        self.overlap = overlap
        self.side = torch.cuda.Stream(device=device) if overlap else None

    def begin(self, seq):
        """seq: list of (codes, bcodes, wscale, N, K) in the order the GEMMs run."""
        self.seq, self._joined = seq, None
        ng = -(-len(seq) // self.group)
        self.ready, self.done = [None] * ng, [None] * ng
        self.main = torch.cuda.current_stream()
        if self.overlap:
            self.side.wait_stream(self.main)
            self._decode_group(0)

    def _view(self, g):
        _, _, _, N, K = self.seq[g]
        j, p = divmod(g, self.group)
        assert N * K <= self.sizes[p]
        return self.bufs[j % 2][p][:N * K].view(N, K)

    def _decode_group(self, j):
        lo, hi = j * self.group, min((j + 1) * self.group, len(self.seq))
        if not self.overlap:
            for g in range(lo, hi):
                codes, bc, _, N, K = self.seq[g]
                S.unpack_i8(codes, bc, N, K, out=self._view(g))
            return
        with torch.cuda.stream(self.side):
            if j >= 2:
                self.side.wait_event(self.done[j - 2])       # the last GEMM that read this set of buffers
            for g in range(lo, hi):
                codes, bc, _, N, K = self.seq[g]
                S.unpack_i8(codes, bc, N, K, out=self._view(g))
            self.ready[j] = torch.cuda.Event()
            self.ready[j].record(self.side)

    def join(self, g):
        """Make the main stream wait for the decode of g's group and start the next group's decode.  Called by weight() when
        g opens a group; a caller may call it earlier (before the launches that precede the group's first GEMM)."""
        j = g // self.group
        if getattr(self, "_joined", None) == (id(self.seq), j):
            return
        self._joined = (id(self.seq), j)
        if self.overlap:
            if (j + 1) * self.group < len(self.seq):
                self._decode_group(j + 1)                    # overlaps with the GEMMs of group j
            self.main.wait_event(self.ready[j])
        else:
            self._decode_group(j)

    def weight(self, g):
        """INT8 operand of GEMM g; call right before launching it."""
        if g % self.group == 0:
            self.join(g)
        return self._view(g)

    def released(self, g):
        """Call right after launching GEMM g."""
        if self.overlap and (g % self.group == self.group - 1 or g == len(self.seq) - 1):
            self.done[g // self.group] = torch.cuda.Event()
            self.done[g // self.group].record(self.main)

    def end(self):
        self._joined = None
        if self.overlap:
            self.main.wait_stream(self.side)


class DenseStack:
    def __init__(self, layers, M, hidden, eps=1e-6, overlap=True, ring_group=1):
        """layers: list of {group: (codes, bcodes, wscale, N, K)} with gate|up rows already interleaved
        (sc_kernels.interleave_gate_up); M: rows (a multiple of 128); hidden: model width."""
        assert M % S.TM == 0
        self.layers, self.M, self.hidden, self.eps, self.overlap = layers, M, hidden, eps, overlap
        dev = layers[0]["qkv"][0].device
        assert len(GROUPS) % ring_group == 0
        sizes = [max(lw[g][3] * lw[g][4] for lw in layers for g in GROUPS[p::ring_group]) for p in range(ring_group)]
        self.ring = DecodeRing(sizes, dev, overlap, group=ring_group)
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
