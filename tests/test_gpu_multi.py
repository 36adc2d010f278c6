"""GPU: segmented-row kernels (1 GPU) and the tensor-parallel / expert-parallel chains on 2 GPUs (NCCL), which must
reproduce the single-GPU chains bit for bit because row sharding and expert grouping are exact."""
import importlib
import os
import sys

import numpy as np
import pytest
import torch

from helpers import bf16_np, llm_acts, to_bf16_cuda

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("G,M,w", [(2, 200, 1024), (8, 128, 256), (4, 130, 1536)])
def test_segmented_row_kernels(scmx, oracle, G, M, w):
    S = scmx.sc_kernels
    rng = np.random.default_rng(G + M)
    x = llm_acts(rng, M, G * w, oracle)
    seg = to_bf16_cuda(x).view(M, G, w).permute(1, 0, 2).contiguous()
    xq, xs = S.act_quant_seg(seg)
    xq0, xs0 = S.act_quant(to_bf16_cuda(x))
    assert torch.equal(xq, xq0) and torch.equal(xs, xs0)
    nw = to_bf16_cuda(oracle.bf16_round(rng.lognormal(0, 0.3, G * w).astype(np.float32)))
    a, b = S.rmsnorm_quant_seg(seg, nw, 1e-6)
    a0, b0 = S.rmsnorm_quant(to_bf16_cuda(x), nw, 1e-6)
    assert torch.equal(a, a0) and torch.equal(b, b0)


def _worker(rank, world, port, q):
    """Runs _worker_body and reports an exception instead of leaving the peer blocked in a collective."""
    try:
        _worker_body(rank, world, port, q)
    except BaseException as e:   # noqa: BLE001
        import traceback
        q.put((rank, "".join(traceback.format_exception(type(e), e, e.__traceback__))[-1500:]))
        os._exit(1)


def _worker_body(rank, world, port, q):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        pkg = importlib.import_module("mxfp4-int8-m5_b200")
        F, S, P = pkg.sc_format, pkg.sc_kernels, pkg.parallel
        ok = {}
        # ---- tensor-parallel dense stack vs the single-GPU stack
        M, hidden, Fd, layers = 256, 512, 768, 2
        shapes = dict(qkv=(1024, hidden), o=(hidden, hidden), gu=(2 * Fd, hidden), down=(hidden, Fd))
        g = torch.Generator(device="cuda").manual_seed(0)
        full, local = [], []
        for _ in range(layers):
            lf, ll = {}, {}
            for name, (n, k) in shapes.items():
                wt = torch.randn((n, k), generator=g, device="cuda") * 0.02
                if name == "gu":
                    wt = wt[torch.from_numpy(S.interleave_gate_up(n // 2)).cuda()]
                c, b, s, _, _ = F.quantize_device(wt.contiguous(), want_qw=False)
                lf[name] = (c, b, s, n, k)
                ll[name] = P.shard_packed(c, b, s, n, k, rank, world, 4)
            full.append(lf)
            local.append(ll)
        h = torch.randn((M, hidden), generator=g, device="cuda").to(torch.bfloat16)
        o = torch.randn((M, hidden), generator=g, device="cuda").to(torch.bfloat16)
        ref = pkg.fused_dense.DenseStack(full, M, hidden, overlap=True).step(h, o)
        ref2 = pkg.fused_dense.DenseStack(full, M, hidden, overlap=False).step(h, o)
        w = hidden // world
        tp = P.TensorParallelDense(pkg, local, M, hidden)
        out = tp.step(h.view(M, world, w).permute(1, 0, 2).contiguous(), o[:, rank * w:(rank + 1) * w].contiguous())
        ok["tp"] = bool(torch.equal(out.permute(1, 0, 2).reshape(M, hidden), ref)) and bool(torch.equal(ref, ref2))
        # the same stack with store-based all-gathers over peer memory, eagerly and replayed from a CUDA graph
        ptp = P.PeerTensorParallelDense(pkg, local, M, hidden, Fd)
        hs, ol = h.view(M, world, w).permute(1, 0, 2).contiguous(), o[:, rank * w:(rank + 1) * w].contiguous()
        out2 = ptp.step(hs, ol).clone()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            out3 = ptp.step(hs, ol)
        for _ in range(3):
            graph.replay()
        torch.cuda.synchronize()
        ok["peer_tp"] = bool(torch.equal(out2.permute(1, 0, 2).reshape(M, hidden), ref)) and \
            bool(torch.equal(out3.permute(1, 0, 2).reshape(M, hidden), ref))
        # ---- expert-parallel MoE block vs the single-GPU block
        E, k, D, Fm, L = 8, 2, 512, 256, 512
        perm = torch.from_numpy(S.interleave_gate_up(Fm)).cuda()

        def pack(n, kk, tag, e0, e1, p=None):
            cs, bs, ss = [], [], []
            for e in range(e0, e1):
                ge = torch.Generator(device="cuda").manual_seed(1000 * tag + e)
                wt = torch.randn((n, kk), generator=ge, device="cuda") * 0.02
                if p is not None:
                    wt = wt[p]
                c, b, s, _, _ = F.quantize_device(wt.contiguous(), want_qw=False)
                cs.append(c); bs.append(b); ss.append(s)
            return torch.stack(cs), torch.stack(bs), torch.stack(ss)
        blk_full = pkg.fused_moe.MoeBlock(pack(2 * Fm, D, 1, 0, E, perm), pack(D, Fm, 2, 0, E), E, k, D, Fm)
        El = E // world
        blk_loc = pkg.fused_moe.MoeBlock(pack(2 * Fm, D, 1, rank * El, (rank + 1) * El, perm),
                                         pack(D, Fm, 2, rank * El, (rank + 1) * El), El, k, D, Fm)
        hm = torch.randn((L, D), generator=g, device="cuda").to(torch.bfloat16)
        lg = torch.randn((L, E), generator=g, device="cuda")
        lg[:, 5] = -30.0                                           # an expert nobody routes to
        refm = blk_full.step(hm, lg)
        Lr = L // world
        ep = P.ExpertParallelMoe(pkg, blk_loc, E, k)
        outm = ep.step(hm[rank * Lr:(rank + 1) * Lr].contiguous(), lg[rank * Lr:(rank + 1) * Lr].contiguous())
        ok["ep"] = bool(torch.equal(outm, refm[rank * Lr:(rank + 1) * Lr]))
        # ---- the same block with kernel-side dispatch / return over peer memory, eagerly and replayed from a CUDA graph
        pep = P.PeerExpertParallelMoe(pkg, blk_loc, E, k, Lr)
        hl, ll = hm[rank * Lr:(rank + 1) * Lr].contiguous(), lg[rank * Lr:(rank + 1) * Lr].contiguous()
        o1 = pep.step(hl, ll)
        o2 = pep.step(hl, ll)
        torch.cuda.synchronize()
        ok["peer_ep"] = bool(torch.equal(o1, refm[rank * Lr:(rank + 1) * Lr])) and bool(torch.equal(o2, o1))
        # variants: the three ways expert outputs return (default: stores from the down GEMM's epilogue), each with the
        # packed-weight GEMMs (the default at this size) and with the decode-then-GEMM form; and the per-pass expert decode
        assert pep.early_decode and pep.return_mode == "push"
        outs = []
        was_fused = pep.fused
        for mode in ("push", "pull", "kernel"):
            for f in ((was_fused, False) if was_fused else (False,)):
                pep.return_mode, pep.fused = mode, f
                outs.append(pep.step(hl, ll))
        pep.return_mode, pep.fused = "push", was_fused
        pep.early_decode = False
        o5 = pep.step(hl, ll)
        pep.early_decode = True
        o4 = outs[0] if all(torch.equal(outs[0], o) for o in outs[1:]) else outs[0] * float("nan")
        torch.cuda.synchronize()
        ok["peer_ep_variants"] = bool(torch.equal(o4, o1)) and bool(torch.equal(o5, o1))
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            o3 = pep.step(hl, ll)
        for _ in range(3):
            graph.replay()
        torch.cuda.synchronize()
        ok["peer_ep_graph"] = bool(torch.equal(o3, refm[rank * Lr:(rank + 1) * Lr]))
        blk2 = pkg.fused_moe.MoeBlock(blk_full.gu, blk_full.dn, E, k, D, Fm, two_pass=True)
        ok["two_pass"] = bool(torch.equal(blk2.step(hm, lg), refm))
        torch.cuda.synchronize()
        pkg._lib.check_status()
        q.put((rank, ok))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_tensor_and_expert_parallel_match_single_gpu():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, 29651, q)) for r in range(2)]
    for p in procs:
        p.start()
    first = q.get(timeout=150)
    res = dict([first])
    if isinstance(first[1], dict):
        res.update([q.get(timeout=60)])
    for p in procs:
        p.join(20)
        if p.is_alive():
            p.kill()
    want = dict(tp=True, peer_tp=True, ep=True, peer_ep=True, peer_ep_variants=True, peer_ep_graph=True, two_pass=True)
    assert res == {0: want, 1: want}


def test_peer_paths_as_a_world_of_one_rank():
    """The peer-memory tensor-parallel stack and expert-parallel block (dispatch, plan, dynamic gather, grouped GEMMs with the
    row-mapped epilogue in its three return forms, barriers, the gather epilogue of the dense GEMM) run as a world of ONE rank
    on one GPU and equal the single-GPU stack / block bit for bit, eagerly and from a CUDA graph.  The same worker is the
    2-GPU test's; here every box with a single GPU exercises those kernels."""
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    p = ctx.Process(target=_worker, args=(0, 1, 29653, q))
    p.start()
    res = q.get(timeout=200)
    p.join(20)
    if p.is_alive():
        p.kill()
    want = dict(tp=True, peer_tp=True, ep=True, peer_ep=True, peer_ep_variants=True, peer_ep_graph=True, two_pass=True)
    assert res == (0, want)


def test_dense_stack_overlap_equals_serial(scmx):
    """The side-stream weight decode changes scheduling only: results equal the single-stream chain bit for bit, also
    when replayed from a CUDA graph."""
    F, S = scmx.sc_format, scmx.sc_kernels
    M, hidden, Fd = 256, 512, 768
    shapes = dict(qkv=(1024, hidden), o=(hidden, hidden), gu=(2 * Fd, hidden), down=(hidden, Fd))
    g = torch.Generator(device="cuda").manual_seed(0)
    layers = []
    for _ in range(3):
        lw = {}
        for name, (n, k) in shapes.items():
            c, b, s, _, _ = F.quantize_device((torch.randn((n, k), generator=g, device="cuda") * 0.02).contiguous(), want_qw=False)
            lw[name] = (c, b, s, n, k)
        layers.append(lw)
    h = torch.randn((M, hidden), generator=g, device="cuda").to(torch.bfloat16)
    o = torch.randn((M, hidden), generator=g, device="cuda").to(torch.bfloat16)
    a = scmx.fused_dense.DenseStack(layers, M, hidden, overlap=False).step(h, o)
    st = scmx.fused_dense.DenseStack(layers, M, hidden, overlap=True)
    b = st.step(h, o)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        c = st.step(h, o)
    graph.replay()
    torch.cuda.synchronize()
    scmx._lib.check_status()
    assert torch.equal(a, b) and torch.equal(a, c)
    # the ring may also join the decode stream once per 2 or 4 weights (a layer) instead of before every GEMM
    for group in (2, 4):
        for overlap in (True, False):
            d = scmx.fused_dense.DenseStack(layers, M, hidden, overlap=overlap, ring_group=group).step(h, o)
            torch.cuda.synchronize()
            assert torch.equal(a, d), (group, overlap)
    scmx._lib.check_status()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_one_process_two_devices(scmx):
    """One process driving two GPUs: per-device set-up (shared-memory limits, SM counts, tables) is kept per device, so
    the GEMM with > 48 KB of shared memory, the SwiGLU table and the streaming GEMV work on the second device too."""
    S, G, F = scmx.sc_kernels, scmx.sc_decode, scmx.sc_format
    outs = []
    for dev in (0, 1):
        with torch.cuda.device(dev):
            g = torch.Generator(device=f"cuda:{dev}").manual_seed(3)
            xq = torch.randint(-127, 128, (256, 1024), dtype=torch.int8, device=f"cuda:{dev}", generator=g)
            wq = torch.randint(-96, 97, (512, 1024), dtype=torch.int8, device=f"cuda:{dev}", generator=g)
            xs = torch.rand(256, device=f"cuda:{dev}", generator=g) * 1e-2
            ws = torch.rand(512, device=f"cuda:{dev}", generator=g) * 1e-2
            acc = S.mm_i8_i32(xq, wq)
            y3 = S.mm_epi(xq, wq, xs, ws, 3)
            w = torch.randn((1024, 2048), device=f"cuda:{dev}", generator=g) * 0.02
            c, b, s, _, _ = F.quantize_device(w, want_qw=False)
            scmx._lib.call("scmx_set_gemv_stream", 2)
            try:
                yv = G.gemv(xq[0].repeat(2), c, b, xs[:1], s, 1024, 1)
            finally:
                scmx._lib.call("scmx_set_gemv_stream", 1)
            torch.cuda.synchronize()
            scmx._lib.check_status()
            assert torch.equal(acc, torch._int_mm(xq, wq.t().contiguous()))
            outs.append((acc.cpu(), y3.cpu(), yv.cpu()))
    for a, b in zip(*outs):
        assert torch.equal(a, b)
