"""Multi-GPU forms of the W4A8 path: one process per GPU, torch.distributed (NCCL over NVLink) for the exchanges.

  * Dense layers shard by OUTPUT COLUMN (weight rows).  The format is per output row, so a row slice of codes / bcodes /
    wscale is an exact shard and every rank's INT32 accumulators equal the corresponding columns of the single-GPU GEMM.
    Column shards of a GEMM output are all-gathered into the segment layout [G, M, N/G] and consumed in place by the
    segmented row kernels (act_quant_seg / rmsnorm_quant_seg): no transposing copies, and the residual slice of rank g
    is the contiguous segment g.
  * MoE layers shard by EXPERT, tokens by rank.  Rows are counting-sorted by global expert id (= by destination rank),
    exchanged with all-to-all (INT8 rows + f32 scales out, bf16 rows back), regrouped by local expert on the receiver,
    and returned to the sender in its original sorted order, where moe_combine finishes the block.

The reference is single-device (one Apple GPU, no collectives); the exactness argument for row sharding is the one it
uses for row concatenation (e2e/fused_qwen3.py:36,44-46) and for order independence of the sorted rows
(e2e/sc_moe.py:110-113).  The bookkeeping in this file is device-agnostic so that it also runs on CPU tensors with the
gloo backend.
"""
import ctypes

import torch
import torch.distributed as dist


# ---- host-side bookkeeping (no kernels) ---------------------------------------------------------------------------
def shard_rows(N, rank, world, multiple=1):
    """[r0, r1) of an N-row weight for `rank`; shards are equal and a multiple of `multiple` rows."""
    assert N % (world * multiple) == 0, f"N={N} is not divisible into {world} shards of a multiple of {multiple} rows"
    per = N // world
    return rank * per, (rank + 1) * per


def shard_packed(codes, bcodes, wscale, N, K, rank, world, multiple=1):
    """Row shard of a packed matrix (codes [N*K/8], bcodes [N, ...], wscale [N]) -> (codes, bcodes, wscale, N_local, K)."""
    r0, r1 = shard_rows(N, rank, world, multiple)
    c = codes.reshape(N, K // 8)[r0:r1].reshape(-1).contiguous()
    return c, bcodes[r0:r1].contiguous(), wscale[r0:r1].contiguous(), r1 - r0, K


def expert_owner_splits(cnt, world):
    """cnt int [E] rows per global expert (experts are owned in contiguous blocks of E/world) -> rows per destination rank."""
    return cnt.reshape(world, -1).sum(1)


def exchange_counts(cnt, world, group=None):
    """Every rank sends the counts of the experts owned by rank d to rank d; returns int64 [world, E/world], row s = what
    rank s will send here."""
    send = cnt.reshape(world, -1).to(torch.int64).contiguous()
    recv = torch.empty_like(send)
    dist.all_to_all_single(recv, send, group=group)
    return recv


def exchange_rows(rows, send_splits, recv_splits, group=None, out=None):
    """Variable all-to-all of the leading dimension: rows[sum(send_splits), ...] -> [sum(recv_splits), ...]."""
    n = int(sum(recv_splits))
    if out is None:
        out = torch.empty((n,) + tuple(rows.shape[1:]), dtype=rows.dtype, device=rows.device)
    dist.all_to_all_single(out[:n], rows, output_split_sizes=list(recv_splits), input_split_sizes=list(send_splits), group=group)
    return out


def local_expert_ids(recv_cnt):
    """recv_cnt int64 [world, El] -> local expert id of every received row (rows arrive source-major, expert-minor)."""
    world, El = recv_cnt.shape
    ids = torch.arange(El, device=recv_cnt.device, dtype=torch.int32).repeat(world)
    return torch.repeat_interleave(ids, recv_cnt.reshape(-1), output_size=int(recv_cnt.sum()))


# ---- tensor-parallel dense stack ----------------------------------------------------------------------------------------
class TensorParallelDense:
    """Column-sharded dense decoder stack (see fused_dense.DenseStack for the chain)."""

    def __init__(self, pkg, layers_local, M, hidden, group=None, eps=1e-6):
        """layers_local: this rank's row shards {group: (codes, bcodes, wscale, N_local, K)} (shard_packed)."""
        self.S, self.layers, self.M, self.hidden, self.eps, self.group = pkg.sc_kernels, layers_local, M, hidden, eps, group
        self.pkg_lib = pkg._lib
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        dev = layers_local[0]["qkv"][0].device
        self.nw = torch.ones(hidden, dtype=torch.bfloat16, device=dev)
        self.launches_per_layer = 12

    def gather(self, local):
        """[M, w] column shard -> [G, M, w] segment layout on every rank."""
        out = torch.empty((self.world,) + tuple(local.shape), dtype=local.dtype, device=local.device)
        dist.all_gather_into_tensor(out.view(-1, local.shape[1]), local.contiguous(), group=self.group)
        return out

    def _gemm(self, lw, name, xq, xs, epi, res=None):
        codes, bc, ws, n, k = lw[name]
        return self.S.mm_epi(xq, self.S.unpack_i8(codes, bc, n, k), xs, ws, epi, res=res)

    def step(self, h_seg, o_local):
        """h_seg bf16 [G, M, hidden/G]: residual stream in segment layout; o_local bf16 [M, hidden/G]: this rank's columns
        of the attention output.  Returns the new residual stream, again in segment layout (identical on every rank)."""
        S, M, r = self.S, self.M, self.rank
        for lw in self.layers:
            xq, xs = S.rmsnorm_quant_seg(h_seg, self.nw, self.eps, M)
            self._gemm(lw, "qkv", xq, xs, 1)                       # this rank's heads; attention is outside the path
            oq, os_ = S.act_quant_seg(self.gather(o_local), M)
            h_seg = self.gather(self._gemm(lw, "o", oq, os_, 2, res=h_seg[r]))
            xq, xs = S.rmsnorm_quant_seg(h_seg, self.nw, self.eps, M)
            act = self._gemm(lw, "gu", xq, xs, 3)                  # [M, F/G]
            aq, as_ = S.act_quant_seg(self.gather(act), M)
            h_seg = self.gather(self._gemm(lw, "down", aq, as_, 2, res=h_seg[r]))
        return h_seg


# ---- expert-parallel MoE half-block -----------------------------------------------------------------------------------------
class ExpertParallelMoe:
    """MoE half-block with experts [rank*E/G, (rank+1)*E/G) on this rank and L/G tokens per rank."""

    def __init__(self, pkg, block_local, n_experts, topk, group=None):
        """block_local: fused_moe.MoeBlock built from this rank's E/G experts."""
        self.pkg, self.block, self.E, self.k, self.group = pkg, block_local, n_experts, topk, group
        self.world = dist.get_world_size(group)
        assert n_experts % self.world == 0 and block_local.E == n_experts // self.world

    def step(self, h, logits):
        """h bf16 [Lr, D] local tokens, logits f32 [Lr, E] over ALL experts -> new residual rows bf16 [Lr, D]."""
        S, M_, L_ = self.pkg.sc_kernels, self.pkg.sc_moe, self.pkg._lib
        blk, G, k = self.block, self.world, self.k
        Lr, D = h.shape
        R = Lr * k
        xq, xs = S.rmsnorm_quant(h, blk.nw, blk.eps, Lr)
        inds, scores = M_.router_topk(logits, k)
        pos, tok, _, off, _, _ = M_.route_sort(inds, self.E, M_.TM)      # sorted by global expert = by destination rank
        xq_s, xs_s = M_.gather_rows(xq, xs, tok, R)
        cnt = off[1:] - off[:-1]
        recv_cnt = exchange_counts(cnt, G, self.group)
        splits = torch.stack([expert_owner_splits(cnt.to(torch.int64), G), recv_cnt.sum(1)]).cpu()   # the one host sync
        send_splits, recv_splits = splits[0].tolist(), splits[1].tolist()
        Rr = int(sum(recv_splits))
        rx_q = torch.empty((Rr + M_.TM, D), dtype=torch.int8, device=h.device)
        exchange_rows(xq_s[:R], send_splits, recv_splits, self.group, out=rx_q)
        rx_s = exchange_rows(xs_s, send_splits, recv_splits, self.group)
        # regroup the received rows by local expert
        le = local_expert_ids(recv_cnt)
        pos2, tok2, _, off2, ts2, mt2 = M_.route_sort(le.view(Rr, 1), blk.E, M_.TM)
        xq_r, xs_r = M_.gather_rows(rx_q, rx_s, tok2, Rr)
        y_sorted = blk.experts(xq_r, xs_r, Rr, off2, ts2, mt2)             # bf16 [Rr, D]
        # back to arrival order (row i of the receive buffer is sorted row pos2[i]), then back to the senders
        y_rx = torch.empty((Rr, D), dtype=torch.bfloat16, device=h.device)
        if Rr:
            L_.call("scmx_gather_rows", L_.ptr(y_sorted.view(torch.int8)), None, L_.ptr(pos2), Rr, 0, 2 * D,
                    L_.ptr(y_rx.view(torch.int8)), None, L_.stream())
        y_back = exchange_rows(y_rx, recv_splits, send_splits, self.group)
        hout, _, _ = M_.moe_combine(y_back, pos, scores, h, blk.nw, blk.eps, Lr, quant=False)
        return hout


# ---- expert parallelism over peer memory (no host round trip, capturable in a CUDA graph) -------------------------------
def _lib_enable_peer(peer_device):
    from . import _lib
    _lib.call("scmx_enable_peer_access", int(peer_device))


def share_tensor(t, group=None):
    """Every rank passes its own CUDA tensor `t` (same shape and dtype everywhere); returns the list of all ranks' tensors
    as seen from this process: entry `rank` is `t` itself, the others are CUDA-IPC mappings of the peers' memory."""
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    meta = (t.untyped_storage()._share_cuda_(), t.storage_offset(), tuple(t.shape), t.dtype)
    metas = [None] * world
    dist.all_gather_object(metas, meta, group=group)
    views = []
    for r, (m, off, shape, dtype) in enumerate(metas):
        if r == rank:
            views.append(t)
            continue
        # Open the peer's allocation with THIS rank's device current: the mapping then belongs to the context the kernels of
        # this rank run in (a mapping opened under the exporter's device index is not addressable from this device).
        me = torch.cuda.current_device()
        dist_dev = m[0]
        if dist_dev != me:
            _lib_enable_peer(dist_dev)
        st = torch.UntypedStorage._new_shared_cuda(me, *m[1:])
        views.append(torch.empty(0, dtype=dtype, device=st.device).set_(st, off, shape))
    return views


class PeerExpertParallelMoe:
    """ExpertParallelMoe whose dispatch and return are kernels storing into peer GPUs' memory (scmx_ep_*): the counts never
    visit the host, so the whole half-block is one stream of launches and can be replayed from a CUDA graph."""

    def __init__(self, pkg, block_local, n_experts, topk, tokens_local, group=None):
        import ctypes
        self.pkg, self.block, self.E, self.k, self.group = pkg, block_local, n_experts, topk, group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        assert n_experts % self.world == 0 and block_local.E == n_experts // self.world and self.world <= 8
        L_ = pkg._lib
        dev = block_local.nw.device
        G, D, El, TM = self.world, block_local.D, block_local.E, pkg.sc_moe.TM
        self.Lr, self.cap = tokens_local, tokens_local * topk
        self.r_cap = G * self.cap
        i32 = dict(dtype=torch.int32, device=dev)
        self.rx_q = torch.empty((G, self.cap, D), dtype=torch.int8, device=dev)
        self.rx_s = torch.empty((G, self.cap), dtype=torch.float32, device=dev)
        self.rx_meta = torch.zeros((G, El + 1), **i32)
        self.y_back = torch.empty((self.cap, D), dtype=torch.bfloat16, device=dev)
        self.flags = torch.zeros(G, **i32)
        self.epoch = torch.zeros(1, **i32)
        torch.cuda.synchronize()
        self._views = {}
        self._peers = {}
        # "pull" return: expert outputs stay here, ordered by receive slot; the token's owner reads them in its combine
        self.y_slot = torch.empty((G * self.cap, D), dtype=torch.bfloat16, device=dev)
        self.zero_rank = torch.zeros(G * self.cap + TM, **i32)
        self._own_slot = (ctypes.c_void_p * 8)(self.y_slot.data_ptr(), *([None] * 7))
        for name in ("rx_q", "rx_s", "rx_meta", "y_back", "flags", "y_slot"):
            views = share_tensor(getattr(self, name), group)
            self._views[name] = views                      # keep the mappings alive
            self._peers[name] = (ctypes.c_void_p * 8)(*[v.data_ptr() for v in views], *([None] * (8 - G)))
        dist.barrier(group)
        # With few experts per rank the whole rank's expert weights decode to a modest INT8 buffer: the decode is started on a
        # side stream at the top of every step and overlaps routing, dispatch and the barrier (weights do not depend on them).
        F = block_local.F
        self.early_decode = El * 3 * F * D <= (1 << 30)
        # How expert outputs travel back to the token's owner:
        #   "push"   the down GEMM's epilogue stores every output row straight into the owner's buffer over NVLink (full
        #            128-byte lines from the staged epilogue), so the transfer overlaps the GEMM; barrier; local combine.
        #   "pull"   the down GEMM stores its rows by receive slot in a local buffer; barrier; every rank's combine loads
        #            the rows of its tokens from the owners over peer memory.
        #   "kernel" plain GEMM, then a return kernel (scmx_ep_return) storing whole rows; barrier; local combine.
        # Measured on 2 GPUs, 4096 tokens per GPU: push 0.544 ms, pull 0.580 ms, kernel 0.611 ms (4096 tokens in total:
        # 0.339 / 0.362 / 0.374 ms).  All three give the same bits.
        self.return_mode = "push"
        # fused: the grouped GEMMs read the packed expert weights and expand them inside the kernel (scmx_moe_mm_w4): no per-step
        # decode launches and no INT8 copy.  Per rank the block is a chain of short kernels, where two launches fewer count.
        self.fused = bool(pkg.sc_moe.FUSED_UNPACK and block_local.E <= 512 and
                          L_.lib().scmx_w4_supported(pkg.sc_format.DEFAULT.c_struct(), D) and
                          L_.lib().scmx_w4_supported(pkg.sc_format.DEFAULT.c_struct(), block_local.F))
        self.fmt = pkg.sc_format.DEFAULT
        if self.early_decode:
            self.side = torch.cuda.Stream(device=dev)
            self.gu8 = torch.empty((El * 2 * F, D), dtype=torch.int8, device=dev)
            self.dn8 = torch.empty((El * D, F), dtype=torch.int8, device=dev)
        self.route_stream = torch.cuda.Stream(device=dev)
        self.off2 = torch.empty(El + 1, **i32)
        self.ts2 = torch.empty(El + 1, **i32)
        self.tok2 = torch.empty(self.r_cap + TM, **i32)
        self.ret_rank = torch.empty(self.r_cap, **i32)
        self.ret_row = torch.empty(self.r_cap, **i32)
        self.n_rows = torch.zeros(1, **i32)

    def _barrier(self):
        L_ = self.pkg._lib
        L_.call("scmx_peer_barrier", self._peers["flags"], self.rank, self.world, L_.ptr(self.epoch), L_.ptr(L_.status_buffer()),
                L_.stream())

    def step(self, h, logits):
        """h bf16 [Lr, D] local tokens, logits f32 [Lr, E] -> new residual rows bf16 [Lr, D]."""
        S, M_, L_ = self.pkg.sc_kernels, self.pkg.sc_moe, self.pkg._lib
        blk, G, k = self.block, self.world, self.k
        Lr, D = h.shape
        assert Lr == self.Lr
        R, TM, F = Lr * k, M_.TM, blk.F
        # packed-weight GEMMs only where a local expert sees few rows (expected rows per expert = tokens * topk / experts)
        fused = self.fused and self.early_decode and (Lr * k * G) // self.E < blk.FUSED_BELOW
        if self.early_decode and not fused:
            main = torch.cuda.current_stream()
            self.side.wait_stream(main)
            with torch.cuda.stream(self.side):
                S.unpack_i8(blk.gu[0].reshape(-1), blk.gu[1].reshape(blk.E * 2 * F, -1), blk.E * 2 * F, D, out=self.gu8)
                S.unpack_i8(blk.dn[0].reshape(-1), blk.dn[1].reshape(blk.E * D, -1), blk.E * D, F, out=self.dn8)
                decoded = torch.cuda.Event()
                decoded.record(self.side)
        # routing (top-k, counting sort) does not depend on the quantized rows: it runs beside RMSNorm + INT8 on a stream of its own
        cur = torch.cuda.current_stream()
        self.route_stream.wait_stream(cur)
        with torch.cuda.stream(self.route_stream):
            inds, scores = M_.router_topk(logits, k)
            pos, tok, es, off, _, _ = M_.route_sort(inds, self.E, TM)
        xq, xs = S.rmsnorm_quant(h, blk.nw, blk.eps, Lr)
        cur.wait_stream(self.route_stream)
        L_.call("scmx_ep_dispatch", L_.ptr(xq), L_.ptr(xs), L_.ptr(tok), L_.ptr(es), L_.ptr(off), R, D, self.E, G, self.rank, self.cap,
                self._peers["rx_q"], self._peers["rx_s"], self._peers["rx_meta"], L_.stream())
        self._barrier()
        L_.call("scmx_ep_plan", L_.ptr(self.rx_meta), G, blk.E, self.cap, TM, self.r_cap, L_.ptr(self.off2), L_.ptr(self.ts2),
                L_.ptr(self.tok2), L_.ptr(self.ret_rank), L_.ptr(self.ret_row), L_.ptr(self.n_rows), L_.stream())
        xq_r = torch.empty((self.r_cap + TM, D), dtype=torch.int8, device=h.device)
        xs_r = torch.empty(self.r_cap + TM, dtype=torch.float32, device=h.device)
        L_.call("scmx_gather_rows_dyn", L_.ptr(self.rx_q), L_.ptr(self.rx_s), L_.ptr(self.tok2), L_.ptr(self.n_rows), self.r_cap, TM, D,
                L_.ptr(xq_r), L_.ptr(xs_r), L_.stream())
        mt = -(-self.r_cap // TM) + blk.E
        if fused or not self.early_decode:
            act = M_.moe_mm(xq_r, self.r_cap, *blk.gu, self.off2, self.ts2, mt, 2 * F, 3, xs_r)
        else:
            main.wait_event(decoded)
            act = M_.moe_mm_i8(xq_r, self.r_cap, self.gu8, blk.gu[2], self.off2, self.ts2, mt, 2 * F, 3, xs_r)
        xq2 = torch.empty((self.r_cap + TM, F), dtype=torch.int8, device=h.device)
        xs2 = torch.empty(self.r_cap + TM, dtype=torch.float32, device=h.device)
        L_.call("scmx_act_quant_dyn", L_.ptr(act), L_.ptr(self.n_rows), self.r_cap, TM, F, L_.ptr(xq2), L_.ptr(xs2), L_.stream())
        mode = self.return_mode if self.early_decode else "kernel"
        if mode == "kernel":
            if fused or not self.early_decode:
                yd = M_.moe_mm(xq2, self.r_cap, *blk.dn, self.off2, self.ts2, mt, D, 1, xs2)
            else:
                yd = M_.moe_mm_i8(xq2, self.r_cap, self.dn8, blk.dn[2], self.off2, self.ts2, mt, D, 1, xs2)
            L_.call("scmx_ep_return", L_.ptr(yd), L_.ptr(self.ret_rank), L_.ptr(self.ret_row), L_.ptr(self.n_rows), self.r_cap, D, G,
                    self._peers["y_back"], L_.stream())
        else:
            # the down GEMM with a row-mapped epilogue: into the owners' y_back (push) or by receive slot into y_slot (pull)
            if mode == "push":
                rr, rw, world, dst = self.ret_rank, self.ret_row, G, self._peers["y_back"]
            else:
                rr, rw, world, dst = self.zero_rank, self.tok2, 1, self._own_slot
            if fused:
                L_.call("scmx_moe_mm_w4_ret", L_.ptr(xq2), self.r_cap, L_.ptr(blk.dn[0]), L_.ptr(blk.dn[1]), L_.ptr(blk.dn[2]),
                        L_.ptr(self.off2), blk.E, D, F, self.fmt.c_struct(), L_.ptr(xs2), L_.ptr(rr), L_.ptr(rw), world, dst,
                        L_.ptr(L_.status_buffer()), L_.stream())
            else:
                L_.call("scmx_moe_mm_i8_ret", L_.ptr(xq2), self.r_cap, L_.ptr(self.dn8), L_.ptr(blk.dn[2]), L_.ptr(self.off2),
                        L_.ptr(self.ts2), blk.E, D, F, L_.ptr(xs2), L_.ptr(rr), L_.ptr(rw), world, dst, TM,
                        L_.ptr(L_.status_buffer()), L_.stream())
        self._barrier()
        if mode == "pull":
            hout = torch.empty((Lr, D), dtype=torch.bfloat16, device=h.device)
            L_.call("scmx_moe_combine_pull", self._peers["y_slot"], G, self.rank, blk.E, self.cap, L_.ptr(es), L_.ptr(off), L_.ptr(pos),
                    L_.ptr(scores), L_.ptr(h), L_.ptr(blk.nw), float(blk.eps), Lr, Lr, D, k, 0, L_.ptr(hout), None, None, L_.stream())
            return hout
        hout, _, _ = M_.moe_combine(self.y_back, pos, scores, h, blk.nw, blk.eps, Lr, quant=False)
        return hout


class PeerTensorParallelDense(TensorParallelDense):
    """TensorParallelDense whose all-gathers are kernels storing each rank's column shard into every GPU's segment buffer
    (scmx_peer_put + scmx_peer_barrier) instead of library collectives: the whole stack is one stream of launches and can be
    replayed from a CUDA graph.  Two residual buffers alternate so that a gather never overwrites rows a peer still reads."""

    def __init__(self, pkg, layers_local, M, hidden, ffn, group=None, eps=1e-6):
        import ctypes
        super().__init__(pkg, layers_local, M, hidden, group, eps)
        G = self.world
        dev = self.nw.device
        bf = dict(dtype=torch.bfloat16, device=dev)
        self.bufs = dict(o=torch.empty((G, M, hidden // G), **bf), h0=torch.empty((G, M, hidden // G), **bf),
                         h1=torch.empty((G, M, hidden // G), **bf), act=torch.empty((G, M, ffn // G), **bf),
                         flags=torch.zeros(G, dtype=torch.int32, device=dev))
        self.epoch = torch.zeros(1, dtype=torch.int32, device=dev)
        torch.cuda.synchronize()
        self._views, self._peers = {}, {}
        for name, t in self.bufs.items():
            views = share_tensor(t, group)
            self._views[name] = views
            self._peers[name] = (ctypes.c_void_p * 8)(*[v.data_ptr() for v in views], *([None] * (8 - G)))
        dist.barrier(group)

    def gather_to(self, local, name):
        """Column shard [M, w] -> the shared segment buffer `name` [G, M, w], complete on every rank when this returns
        (in stream order)."""
        L_ = self.pkg_lib
        nbytes = local.numel() * local.element_size()
        L_.call("scmx_peer_put", L_.ptr(local), nbytes, self.rank * nbytes, self._peers[name], self.world, L_.stream())
        self._barrier()
        return self.bufs[name]

    def _barrier(self):
        L_ = self.pkg_lib
        L_.call("scmx_peer_barrier", self._peers["flags"], self.rank, self.world, L_.ptr(self.epoch), L_.ptr(L_.status_buffer()),
                L_.stream())

    def _segment_peers(self, name):
        """Host array of pointers: this rank's segment inside every rank's copy of buffer `name`."""
        import ctypes
        if name not in self._seg_peers:
            t = self.bufs[name]
            seg_bytes = t[0].numel() * t.element_size()
            ptrs = [v.data_ptr() + self.rank * seg_bytes for v in self._views[name]]
            self._seg_peers[name] = (ctypes.c_void_p * 8)(*ptrs, *([None] * (8 - self.world)))
        return self._seg_peers[name]

    def _gemm_gather(self, g, xq, xs, epi, name, res=None):
        """GEMM g of the step whose output columns are gathered into segment buffer `name` on every rank.  When the shard is
        wide enough for the CTA-pair kernel the gather is the GEMM's own epilogue (scmx_mm_i8_bcast: full lines stored into every
        GPU's buffer while other tiles compute) and only the barrier follows; otherwise GEMM, store kernel, barrier."""
        L_, S = self.pkg_lib, self.S
        _, _, ws, n, k = self.ring.seq[g]
        wq = self.ring.weight(g)
        M = xq.shape[0]
        n_out = n // 2 if epi == 3 else n
        if self.fused_gather and M > 128 and n >= 256:
            L_.call("scmx_mm_i8_bcast", L_.ptr(xq), L_.ptr(wq), M, n, k, epi, L_.ptr(xs), L_.ptr(ws), L_.ptr(res) if epi == 2 else None,
                    self._segment_peers(name), self.world, L_.ptr(L_.status_buffer()), L_.stream())
            self.ring.released(g)
            self._barrier()
            return self.bufs[name]
        y = S.mm_epi(xq, wq, xs, ws, epi, res=res)
        self.ring.released(g)
        assert y.shape[1] == n_out
        return self.gather_to(y, name)

    def step(self, h_seg, o_local):
        from . import fused_dense as FD
        S, M, r = self.S, self.M, self.rank
        if not hasattr(self, "ring"):
            big = max(n * k for lw in self.layers for (_, _, _, n, k) in lw.values())
            self.ring = FD.DecodeRing(big, self.nw.device, overlap=True)
            self._seg_peers = {}
            self.fused_gather = True
        ring = self.ring
        ring.begin([lw[g] for lw in self.layers for g in FD.GROUPS])
        cur, g = h_seg, 0
        for lw in self.layers:
            xq, xs = S.rmsnorm_quant_seg(cur, self.nw, self.eps, M)
            _, _, ws, n, k = ring.seq[g]
            S.mm_epi(xq, ring.weight(g), xs, ws, 1)               # this rank's heads; attention is outside the path
            ring.released(g)
            oq, os_ = S.act_quant_seg(self.gather_to(o_local, "o"), M)
            nxt = self._gemm_gather(g + 1, oq, os_, 2, "h0", res=cur[r])
            xq, xs = S.rmsnorm_quant_seg(nxt, self.nw, self.eps, M)
            act = self._gemm_gather(g + 2, xq, xs, 3, "act")
            aq, as_ = S.act_quant_seg(act, M)
            cur = self._gemm_gather(g + 3, aq, as_, 2, "h1", res=nxt[r])
            g += 4
        ring.end()
        return cur
