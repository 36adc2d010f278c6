"""Benchmark of the SC-MXFP4 W4A8 hot path on B200.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload dense|moe]

One step = one pass of the hot path over one batch of synthetic input.  Default workload (N = 1): the
Qwen3-1.7B-shaped dense prefill, 28 layers x {qkv 4096x2048, o 2048x2048, gate|up 12288x2048, down 2048x6144} at
M = 2048 tokens, every projection SC-MXFP4-packed from N(0, 0.02) weights; per layer the chain is
rmsnorm_quant -> qkv GEMM (EPI 1) | act_quant -> o GEMM (+residual) -> rmsnorm_quant -> gate|up GEMM (SwiGLU) ->
act_quant -> down GEMM (+residual), each GEMM preceded by the 4-bit -> INT8 weight decode.  The metric is W4A8 GEMM
TOPS = 2 * M * sum(N K) * layers / step time (algorithmic ops only).  The same JSON line also reports the decode GEMV
(GB/s over the 717.9 MB of packed weights) and one OLMoE-shaped MoE half-block (tokens/s).

`--impl reference` times the CPU restatement of the reference's NumPy path (oracle/) on the host cores.
"""
import argparse
import importlib
import json
import os
import subprocess
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

QWEN = dict(layers=28, M=2048, groups=dict(qkv=(4096, 2048), o=(2048, 2048), gu=(12288, 2048), down=(2048, 6144)))
OLMOE = dict(layers=16, tokens=4096, D=2048, F=1024, E=64, topk=8)
# large-MoE stress: 128 experts, block-16 integer-exact FP4 variant (e2m1 / B16 / power-of-two multipliers), Zipf-skewed routing
MOE5 = dict(layers=48, tokens=8192, D=2048, F=768, E=128, topk=8, zipf=1.2, decode_steps=128)


def qwen_ops(M=QWEN["M"], layers=QWEN["layers"]):
    return 2 * M * sum(n * k for n, k in QWEN["groups"].values()) * layers


def gemv_bytes(n, k):
    """Algorithmic bytes of one SC-MXFP4 GEMV: codes + 2-bit block codes + row scales + xq, xs + bf16 out."""
    return n * k // 2 + n * k // 128 + 4 * n + k + 4 + 2 * n


# ------------------------------------------------------------------------------------------------------------------
class ClockSampler:
    """nvidia-smi clock / throttle-reason samples taken while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.idx, self.proc, self.path = gpu_index, None, None

    def __enter__(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms",
                                          "20", "-i", str(self.idx)], stdout=open(self.path, "w"),
                                         stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None
        # nvidia-smi needs up to a second to start (longer on an 8-GPU node): wait for its first line, so that the timed
        # region that follows is sampled from its start; lines written before it are not counted
        self.skip = 0
        if self.proc:
            t0 = time.time()
            while time.time() - t0 < 6.0:
                try:
                    self.skip = sum(1 for _ in open(self.path))
                except OSError:
                    self.skip = 0
                if self.skip:
                    break
                time.sleep(0.02)
        return self

    def __exit__(self, *a):
        if self.proc:
            self.proc.terminate()
            self.proc.wait()

    def summary(self):
        out = dict(sm_mhz=None, sm_max_mhz=None, reasons=[], samples=0)
        if not self.path or not os.path.exists(self.path):
            return out
        sm, mx, reasons = [], [], set()
        lines = open(self.path).read().splitlines()
        if len(lines) > self.skip:             # the samples taken since the timed region began
            lines = lines[self.skip:]
        for line in lines:
            f = [c.strip() for c in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        os.unlink(self.path)
        if sm:
            busy = [s for s in sm if s > 0.5 * max(sm)] or sm
            out.update(sm_mhz=float(np.median(busy)), sm_max_mhz=max(mx), samples=len(sm))
        out["reasons"] = sorted(reasons)
        return out


def peaks():
    p = dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source="fallback")
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        m = json.load(open(path))
        p.update(hbm_gbs=m["hbm_gbs"], bf16_tflops=m["bf16_tflops"],
                 bf16_tflops_sustained=m.get("bf16_tflops_sustained", m["bf16_tflops"]), source="measured")
    return p


# ------------------------------------------------------------------------------------------------------------------
# reference arm / CPU baseline: the oracle's restatement of the reference NumPy path on the host cores
# ------------------------------------------------------------------------------------------------------------------
def cpu_dense_layer_sample(seed=0, M=QWEN["M"]):
    """One Qwen3-1.7B-shaped layer (4 GEMM groups) at M tokens through the oracle: act-quant (float32 recipe), INT32
    GEMM via float64 BLAS, scaling epilogue.  Weights are random INT8 operands in the quantizer's range (packing is
    a load-time step and is not part of the per-step path).  Returns (seconds, ops)."""
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import scmx_oracle as O
    rng = np.random.default_rng(seed)
    ws = {g: (rng.integers(-96, 97, nk).astype(np.int8), np.full(nk[0], 2.0 ** -9, np.float32)) for g, nk in QWEN["groups"].items()}
    xs_in = {g: O.bf16_round(rng.standard_normal((M, nk[1])).astype(np.float32)) for g, nk in QWEN["groups"].items()}
    res = O.bf16_round(rng.standard_normal((M, 2048)).astype(np.float32))
    t0 = time.perf_counter()
    for g, (wq, wsc) in ws.items():
        xq, xs = O.act_quant(xs_in[g])
        acc = O.gemm_i32(xq, wq)
        if g == "gu":
            O.epilogue(acc, xs, wsc, 3)
        elif g == "qkv":
            O.epilogue(acc, xs, wsc, 1)
        else:
            O.epilogue(acc, xs, wsc, 2, res)
    dt = time.perf_counter() - t0
    return dt, qwen_ops(M, 1)


def blas_threads(want=None):
    """Sets the BLAS pool NumPy uses to `want` threads (all host cores by default; a launcher may have exported
    OMP_NUM_THREADS=1) and returns the number the pool then reports."""
    want = want or os.cpu_count() or 1
    try:
        import threadpoolctl
        threadpoolctl.threadpool_limits(limits=want, user_api="blas")
        got = [p.get("num_threads") for p in threadpoolctl.threadpool_info() if p.get("user_api") == "blas"]
        return max(got) if got else 1
    except Exception:   # noqa: BLE001
        return int(os.environ.get("OMP_NUM_THREADS", "0")) or want


def cpu_gemv_sample(seed=0):
    """The reference's CPU check of the decode GEMV (e2e/sc_decode.py:253): qw.astype(int64) @ xq plus the scaling epilogue
    for the four projection groups of ONE layer (25.6 MB of packed weights when stored 4-bit).  Returns (seconds, bytes)."""
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import scmx_oracle as O
    rng = np.random.default_rng(seed)
    ws = {g: (rng.integers(-96, 97, nk).astype(np.int8), np.full(nk[0], 2.0 ** -9, np.float32)) for g, nk in QWEN["groups"].items()}
    xq = {k: rng.integers(-127, 128, k).astype(np.int8) for k in (2048, 6144)}
    t0 = time.perf_counter()
    for g, (wq, wsc) in ws.items():
        O.gemv(xq[wq.shape[1]], np.float32(0.01), wq, wsc, 1)
    dt = time.perf_counter() - t0
    return dt, sum(gemv_bytes(n, k) for n, k in QWEN["groups"].values())


def cpu_moe_sample(seed=0, tokens=512):
    """The reference's CPU check of the grouped GEMM (e2e/sc_moe.py:224-226): a per-expert loop of float64 BLAS products
    over the sorted rows, for gate|up (SwiGLU) and down of an OLMoE-shaped block on `tokens` tokens (top-8 of 64 experts).
    Returns (seconds, tokens)."""
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import scmx_oracle as O
    c = OLMOE
    rng = np.random.default_rng(seed)
    E, D, Fd, k = c["E"], c["D"], c["F"], c["topk"]
    R = tokens * k
    ex = np.sort(rng.integers(0, E, R))
    off = np.concatenate([[0], np.cumsum(np.bincount(ex, minlength=E))]).astype(np.int32)
    gu = [rng.integers(-96, 97, (2 * Fd, D)).astype(np.int8) for _ in range(E)]
    dn = [rng.integers(-96, 97, (D, Fd)).astype(np.int8) for _ in range(E)]
    wsg = [np.full(2 * Fd, 2.0 ** -9, np.float32)] * E
    wsd = [np.full(D, 2.0 ** -9, np.float32)] * E
    x = O.bf16_round(rng.standard_normal((R, D)).astype(np.float32))
    t0 = time.perf_counter()
    xq, xs = O.act_quant(x)
    act = O.moe_mm(xq, R, gu, off, 3, xs, wsg)
    xq2, xs2 = O.act_quant(act)
    O.moe_mm(xq2, R, dn, off, 1, xs2, wsd)
    dt = time.perf_counter() - t0
    return dt, tokens


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = blas_threads()
    times = []
    for i in range(args.warmup + args.steps):
        dt, ops = cpu_dense_layer_sample(seed=i)
        if i >= args.warmup:
            times.append(dt)
    t = float(np.mean(times))
    val = ops / t / 1e12
    line = dict(impl="reference", metric="w4a8_gemm_tops", value=val, unit="TOPS", n_gpus=args.gpus, steps=args.steps,
                warmup=args.warmup, ms_per_step=t * 1e3, higher_is_better=True, scaling="strong", vs_baseline=None,
                dtype="int8", data="synthetic",
                config=dict(workload="qwen3-1.7b-shaped dense prefill, M=2048, SC-MXFP4 W4A8", sample="1 of 28 layers per step"),
                cpu_baseline=dict(value=val, unit="TOPS", cores=cores, kind="port",
                                  sample="one layer (4 GEMM groups) at M=2048 per step: act-quant + f64-BLAS INT32 GEMM + epilogue"),
                e2e=dict(value=val, unit="TOPS", h2d_bytes_per_step=0, d2h_bytes_per_step=0))
    print(json.dumps(line))


# ------------------------------------------------------------------------------------------------------------------
# our arm
# ------------------------------------------------------------------------------------------------------------------
def build_dense_layers(pkg, torch, layers, shard=(0, 1), seed=0):
    """Random-init N(0, 0.02) weights of the Qwen3-1.7B-shaped stack, SC-MXFP4-packed on the GPU; with world > 1 only this
    rank's block of output columns (weight rows) is packed.  Every rank draws the same full matrices (same seed)."""
    F, S, P = pkg.sc_format, pkg.sc_kernels, pkg.parallel
    rank, world = shard
    g = torch.Generator(device="cuda").manual_seed(seed)
    out = []
    for _ in range(layers):
        lw = {}
        for name, (n, k) in QWEN["groups"].items():
            w = torch.randn((n, k), generator=g, device="cuda", dtype=torch.float32) * 0.02
            if name == "gu":     # gate rows then up rows -> interleaved 4-row groups for the SwiGLU epilogue
                w = w[torch.from_numpy(S.interleave_gate_up(n // 2)).cuda()]
            if world > 1:
                r0, r1 = P.shard_rows(n, rank, world, 4)
                w = w[r0:r1]
            codes, bc, ws, _, _ = F.quantize_device(w.contiguous(), want_qw=False)
            lw[name] = (codes, bc, ws, w.shape[0], k)
        out.append(lw)
    return out


def bench_decode(pkg, torch, model, pk, reps=10):
    """Batch-1 decode GEMVs over every packed weight set of the stack, 112 independent GEMVs per pass (717.9 MB, nothing
    L2-resident across a pass).  Headline: the whole pass as ONE persistent launch (sc_decode.GemvList); beside it the same
    pass as 112 launches from a CUDA graph, and per projection group (the reference's table, e2e/tune_07.py:63-66) the
    latency per GEMV and GB/s over the 28 layers' weights of that group."""
    G = pkg.sc_decode
    xq = {k: torch.randint(-127, 128, (k,), dtype=torch.int8, device="cuda") for k in (2048, 6144)}
    xs = torch.full((1,), 0.01, device="cuda")
    res = torch.zeros(2048, dtype=torch.bfloat16, device="cuda")
    EPI = dict(qkv=1, o=2, gu=3, down=2)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def timed(run, n):
        for _ in range(3):
            run()
        torch.cuda.synchronize()
        e0.record()
        for _ in range(n):
            run()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / n

    def jobs_of(names):
        return [(xq[lw[n][4]], lw[n][0], lw[n][1], xs, lw[n][2], lw[n][3], EPI[n], res if EPI[n] == 2 else None)
                for lw in model.layers for n in names]

    nbytes = sum(gemv_bytes(n, k) for lw in model.layers for (_, _, _, n, k) in lw.values())
    n_gemv = 4 * len(model.layers)
    whole = G.GemvList(jobs_of(("qkv", "o", "gu", "down")))
    ms = timed(whole.run, reps)
    out = dict(ms_per_step=ms, gemv_per_step=n_gemv, bytes_per_step=nbytes, gbs=nbytes / ms / 1e6, us_per_gemv=ms * 1e3 / n_gemv,
               hbm_frac=nbytes / ms / 1e6 / pk["hbm_gbs"], launches_per_step=1,
               form="one persistent launch over the list of 112 independent GEMVs (gemv_multi_kernel)")
    groups = {}
    for name in ("qkv", "o", "gu", "down"):
        gl = G.GemvList(jobs_of((name,)))
        gms = timed(gl.run, reps)
        n, k = model.layers[0][name][3], model.layers[0][name][4]
        gb = gemv_bytes(n, k) * len(model.layers)
        groups[name] = dict(N=n, K=k, us_per_gemv=gms * 1e3 / len(model.layers), gbs=gb / gms / 1e6,
                            hbm_frac=gb / gms / 1e6 / pk["hbm_gbs"])
        del gl
    out["groups"] = groups

    # the same pass as one launch per GEMV (programmatic dependent launches replayed from a CUDA graph)
    def one_pass():
        for lw in model.layers:
            for name in ("qkv", "o", "gu", "down"):
                codes, bc, ws, n, k = lw[name]
                G.gemv(xq[k], codes, bc, xs, ws, n, EPI[name], res=res if EPI[name] == 2 else None)
    one_pass()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    try:
        with torch.cuda.graph(g):
            one_pass()
        run = g.replay
    except Exception:
        run = one_pass
    cms = timed(run, reps)
    out["per_call_launches"] = dict(ms_per_step=cms, gbs=nbytes / cms / 1e6, us_per_gemv=cms * 1e3 / n_gemv,
                                    hbm_frac=nbytes / cms / 1e6 / pk["hbm_gbs"], launches_per_step=n_gemv)
    out["kernel_roofline"] = dict(kernel="gemv_multi_kernel", workload="the 112-GEMV pass above", bound="hbm",
                                  algorithmic_bytes_per_launch=nbytes, us_per_launch=ms * 1e3, achieved=nbytes / ms / 1e6,
                                  peak=pk["hbm_gbs"], frac=nbytes / ms / 1e6 / pk["hbm_gbs"], unit="GB/s")
    return out


def build_moe_block(pkg, torch, cfg=OLMOE, shard=(0, 1), seed=0, two_pass=False):
    """One OLMoE-shaped MoE half-block: E experts, gate|up [2F, D] (rows interleaved) and down [D, F] each, N(0, 0.02),
    packed on the GPU.  With world > 1 only this rank's experts are built (all ranks use the same per-expert seeds)."""
    F, S = pkg.sc_format, pkg.sc_kernels
    rank, world = shard
    D, Fd, E = cfg["D"], cfg["F"], cfg["E"]
    perm = torch.from_numpy(S.interleave_gate_up(Fd)).cuda()
    e0, e1 = rank * E // world, (rank + 1) * E // world

    def pack(n, k, tag, p=None):
        cs, bs, ss = [], [], []
        for e in range(e0, e1):
            g = torch.Generator(device="cuda").manual_seed(seed * 100003 + tag * 1009 + e)
            w = torch.randn((n, k), generator=g, device="cuda") * 0.02
            if p is not None:
                w = w[p]
            c, b, s_, _, _ = F.quantize_device(w.contiguous(), want_qw=False)
            cs.append(c); bs.append(b); ss.append(s_)
        return torch.stack(cs), torch.stack(bs), torch.stack(ss)
    # with experts sharded over ranks the expert-parallel layer runs its own early decode of the local experts
    return pkg.fused_moe.MoeBlock(pack(2 * Fd, D, 1, perm), pack(D, Fd, 2), e1 - e0, cfg["topk"], D, Fd, two_pass=two_pass,
                                  early_decode=world == 1)


def zipf_logits(torch, tokens, E, s, seed):
    """Router logits N(0, 1) + log zipf_pmf(rank(e); s) under a seeded permutation of the experts: expert popularity
    follows a Zipf law while every token still draws its own noise.  Returns (logits f32 [tokens, E] on the GPU, perm)."""
    g = torch.Generator(device="cuda").manual_seed(seed)
    perm = torch.randperm(E, generator=g, device="cuda")
    rank = (perm + 1).double()
    logp = (-s * rank.log() - (torch.arange(1, E + 1, device="cuda").double() ** -s).sum().log()).float()
    return torch.randn((tokens, E), generator=g, device="cuda") + logp[None, :], perm


def build_moe5_block(pkg, torch, fmt, shard=(0, 1), seed=0):
    """E experts of gate|up [2F, D] (rows interleaved) and down [D, F], N(0, 0.02), packed by the format-family quantizer
    (row base x per-block multiplier search) on the GPU; every expert its own draw and its own allocation."""
    F, S = pkg.sc_format, pkg.sc_kernels
    c = MOE5
    rank, world = shard
    D, Fd, E = c["D"], c["F"], c["E"]
    perm = torch.from_numpy(S.interleave_gate_up(Fd)).cuda()
    e0, e1 = rank * E // world, (rank + 1) * E // world

    def pack(n, k, tag, p=None):
        cs, bs, ss = [], [], []
        for e in range(e0, e1):
            g = torch.Generator(device="cuda").manual_seed(seed * 100003 + tag * 1009 + e)
            w = torch.randn((n, k), generator=g, device="cuda") * 0.02
            if p is not None:
                w = w[p]
            cc, b, s_, _ = F.family_quantize_device(w.contiguous(), fmt)
            cs.append(cc); bs.append(b); ss.append(s_)
        return torch.stack(cs), torch.stack(bs), torch.stack(ss)
    return pkg.fused_moe.MoeBlock(pack(2 * Fd, D, 1, perm), pack(D, Fd, 2), e1 - e0, c["topk"], D, Fd, early_decode=world == 1)


def bench_moe5(pkg, torch, dist=None, reps=5):
    """Large-MoE stress (128 experts, F = 768, block-16 format family, Zipf(1.2) expert popularity): one half-block at 8192
    prefill tokens (expert parallel when a process group is given) and, on one GPU, the batch-1 gather-GEMV decode step."""
    F, S, M_, G = pkg.sc_format, pkg.sc_kernels, pkg.sc_moe, pkg.sc_decode
    c = MOE5
    world = dist.get_world_size() if dist is not None else 1
    rank = dist.get_rank() if dist is not None else 0
    fmt = F.Format(block=16)
    S.set_format(fmt)
    try:
        blk = build_moe5_block(pkg, torch, fmt, shard=(rank, world))
        Lr = c["tokens"] // world
        layer = blk
        if world > 1:
            layer = pkg.parallel.PeerExpertParallelMoe(pkg, blk, c["E"], c["topk"], Lr)
        g = torch.Generator(device="cuda").manual_seed(1)
        h_all = torch.randn((c["tokens"], c["D"]), generator=g, device="cuda").to(torch.bfloat16)
        lg_all, _ = zipf_logits(torch, c["tokens"], c["E"], c["zipf"], seed=2)
        h, lg = h_all[rank * Lr:(rank + 1) * Lr].contiguous(), lg_all[rank * Lr:(rank + 1) * Lr].contiguous()
        inds, _ = M_.router_topk(lg_all, c["topk"])
        cnt = torch.bincount(inds.reshape(-1).long(), minlength=c["E"]).double()
        per_rank = cnt.view(max(world, 1), -1).sum(1)
        out = dict(tokens=c["tokens"], experts=c["E"], format="e2m1 / block 16 / multipliers 1,2,4,8 (format-family quantizer)",
                   rows_per_expert=dict(max=int(cnt.max()), mean=float(cnt.mean()), min=int(cnt.min())),
                   rows_per_rank=dict(max=int(per_rank.max()), mean=float(per_rank.mean()),
                                      imbalance=float(per_rank.max() / per_rank.mean())))
        for _ in range(3):
            layer.step(h, lg)
        torch.cuda.synchronize()
        pkg._lib.check_status()
        run = lambda: layer.step(h, lg)   # noqa: E731
        try:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                layer.step(h, lg)
            run = graph.replay
        except Exception as e:   # noqa: BLE001
            print(f"# moe5 graph capture unavailable ({type(e).__name__}: {e})", file=sys.stderr)
            torch.cuda.synchronize()
        for _ in range(2):
            run()
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            run()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / reps
        if dist is not None:
            t = torch.tensor([ms], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        ops = 2 * c["tokens"] * c["topk"] * 3 * c["F"] * c["D"]
        out.update(ms_per_half_block=ms, tokens_per_s_one_layer=c["tokens"] / ms * 1e3,
                   tokens_per_s_48_layers=c["tokens"] / (ms * c["layers"]) * 1e3, tops=ops / ms / 1e9,
                   parallelism="single GPU" if world == 1 else f"ep{world}: {c['E'] // world} experts and {Lr} tokens per GPU")
        pkg._lib.check_status()
        if world == 1:
            # batch-1 decode of the same layer: RMSNorm + INT8 of one row, router, gather-GEMV over the 8 chosen experts
            # (gate|up with SwiGLU, then down on per-slot rows), weighted combine; 128 steps with fresh logits each
            nw = torch.ones(c["D"], dtype=torch.bfloat16, device="cuda")
            pos = torch.arange(c["topk"], dtype=torch.int32, device="cuda")
            lg1, _ = zipf_logits(torch, c["decode_steps"], c["E"], c["zipf"], seed=3)
            x1 = torch.randn((c["decode_steps"], 1, c["D"]), generator=g, device="cuda").to(torch.bfloat16)

            def step(i):
                xq, xs = S.rmsnorm_quant(x1[i], nw, 1e-5, 1)
                ind1, sc1 = M_.router_topk(lg1[i:i + 1], c["topk"])
                e = ind1.reshape(-1)
                act = G.gemv(xq, blk.gu[0], blk.gu[1], xs, blk.gu[2], 2 * c["F"], 3, eidx=e, xstride=0)
                yd = G.gemv(act, blk.dn[0], blk.dn[1], None, blk.dn[2], c["D"], 1, eidx=e, xstride=1, pro=1)
                return M_.moe_combine(yd, pos, sc1, x1[i], nw, 1e-5, 1, quant=False)[0]
            step(0)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                for i in range(c["decode_steps"]):
                    step(i)
            graph.replay()
            torch.cuda.synchronize()
            e0.record()
            for _ in range(3):
                graph.replay()
            e1.record()
            torch.cuda.synchronize()
            us = e0.elapsed_time(e1) / 3 / c["decode_steps"] * 1e3
            nb = c["topk"] * (gemv_bytes_fmt(2 * c["F"], c["D"], 16, 2) + gemv_bytes_fmt(c["D"], c["F"], 16, 2))
            out["decode"] = dict(steps=c["decode_steps"], us_per_step_one_layer=us, packed_bytes_per_step=nb, gbs=nb / us / 1e3,
                                 form="gather-GEMV over the 8 routed experts (register kernel, expert ids read on the device)")
            pkg._lib.check_status()
        return out
    finally:
        S.set_format(F.Format())


def gemv_bytes_fmt(n, k, block, bc_bits):
    return n * k // 2 + n * k * bc_bits // (8 * block) + 4 * n + k + 4 + 2 * n


def bench_moe(pkg, torch, dist=None, reps=5, weak=False, blk=None, tokens=None):
    """OLMoE-shaped MoE half-block at 4096 tokens: quant -> route -> (dispatch) -> two grouped GEMMs -> (return) -> combine.
    With a process group: experts sharded by rank, tokens split by rank, dispatch and return over NVLink.
    weak: 4096 tokens PER RANK instead of in total."""
    c = dict(OLMOE)
    if tokens:
        c["tokens"] = tokens
    world = dist.get_world_size() if dist is not None else 1
    rank = dist.get_rank() if dist is not None else 0
    if weak:
        c["tokens"] = c["tokens"] * world
    blk = blk if blk is not None else build_moe_block(pkg, torch, shard=(rank, world))
    Lr = c["tokens"] // world
    exchange = "none"
    if world > 1:
        try:
            layer = pkg.parallel.PeerExpertParallelMoe(pkg, blk, c["E"], c["topk"], Lr)
            exchange = "dispatch by stores into peer memory, expert outputs returned by stores from the down GEMM's epilogue, CUDA graph"
        except Exception as e:   # noqa: BLE001
            print(f"# peer-memory path unavailable ({type(e).__name__}: {e}); using NCCL all-to-all, eager launches", file=sys.stderr)
            layer = pkg.parallel.ExpertParallelMoe(pkg, blk, c["E"], c["topk"])
            exchange = "NCCL all-to-all, eager launches"
    else:
        layer = blk
    g = torch.Generator(device="cuda").manual_seed(1)
    h = torch.randn((c["tokens"], c["D"]), generator=g, device="cuda").to(torch.bfloat16)[rank * Lr:(rank + 1) * Lr].contiguous()
    logits = torch.randn((c["tokens"], c["E"]), generator=g, device="cuda")[rank * Lr:(rank + 1) * Lr].contiguous()
    for _ in range(3):
        layer.step(h, logits)
    torch.cuda.synchronize()
    pkg._lib.check_status()
    run = lambda: layer.step(h, logits)   # noqa: E731
    if world == 1 or exchange.startswith("dispatch"):
        try:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                layer.step(h, logits)
            run = graph.replay
        except Exception as e:   # noqa: BLE001
            print(f"# MoE graph capture unavailable ({type(e).__name__}: {e})", file=sys.stderr)
            torch.cuda.synchronize()
    for _ in range(2):
        run()
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.profiler.start()            # a profiler given --profile-from-start off sees the timed passes only
    e0.record()
    for _ in range(reps):
        run()
    e1.record()
    torch.cuda.synchronize()
    torch.cuda.profiler.stop()
    ms = e0.elapsed_time(e1) / reps
    if dist is not None:
        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    ops = 2 * c["tokens"] * c["topk"] * 3 * c["F"] * c["D"]
    return dict(ms_per_half_block=ms, tokens=c["tokens"], tokens_per_s_one_layer=c["tokens"] / ms * 1e3,
                tokens_per_s_16_layers=c["tokens"] / (ms * c["layers"]) * 1e3, tops=ops / ms / 1e9,
                parallelism="single GPU" if world == 1 else f"ep{world}: {c['E'] // world} experts and {Lr} tokens per GPU, {exchange}")


def parity_multi(pkg, torch, dist):
    """Correctness evidence at world > 1, before any timing: a small tensor-parallel dense stack and a small
    expert-parallel MoE block, each compared bit for bit with the single-GPU result computed on every rank (row sharding
    and expert grouping are exact).  Returns {"tp": bool, "ep": bool}, true only if every rank agrees."""
    F, S, P = pkg.sc_format, pkg.sc_kernels, pkg.parallel
    rank, world = dist.get_rank(), dist.get_world_size()
    ok = {}
    M, hidden, Fd, layers = 256, 1024, 1536, 2
    shapes = dict(qkv=(2048, hidden), o=(hidden, hidden), gu=(2 * Fd, hidden), down=(hidden, Fd))
    g = torch.Generator(device="cuda").manual_seed(0)
    full, local = [], []
    for _ in range(layers):
        lf, ll = {}, {}
        for name, (n, k) in shapes.items():
            wt = torch.randn((n, k), generator=g, device="cuda") * 0.02
            if name == "gu":
                wt = wt[torch.from_numpy(S.interleave_gate_up(n // 2)).cuda()]
            c, b, s_, _, _ = F.quantize_device(wt.contiguous(), want_qw=False)
            lf[name] = (c, b, s_, n, k)
            ll[name] = P.shard_packed(c, b, s_, n, k, rank, world, 4)
        full.append(lf)
        local.append(ll)
    h = torch.randn((M, hidden), generator=g, device="cuda").to(torch.bfloat16)
    o = torch.randn((M, hidden), generator=g, device="cuda").to(torch.bfloat16)
    ref = pkg.fused_dense.DenseStack(full, M, hidden, overlap=False).step(h, o)
    w = hidden // world
    hs, ol = h.view(M, world, w).permute(1, 0, 2).contiguous(), o[:, rank * w:(rank + 1) * w].contiguous()
    try:
        tp = P.PeerTensorParallelDense(pkg, local, M, hidden, Fd)
    except Exception:   # noqa: BLE001
        tp = P.TensorParallelDense(pkg, local, M, hidden)
    out = tp.step(hs, ol)
    ok["tp"] = bool(torch.equal(out.permute(1, 0, 2).reshape(M, hidden), ref))
    E, k, D, Fm, L = 8 * max(1, world // 8), 2, 512, 256, 128 * world
    perm = torch.from_numpy(S.interleave_gate_up(Fm)).cuda()

    def pack(n, kk, tag, e0, e1, p=None):
        cs, bs, ss = [], [], []
        for e in range(e0, e1):
            ge = torch.Generator(device="cuda").manual_seed(1000 * tag + e)
            wt = torch.randn((n, kk), generator=ge, device="cuda") * 0.02
            if p is not None:
                wt = wt[p]
            c, b, s_, _, _ = F.quantize_device(wt.contiguous(), want_qw=False)
            cs.append(c); bs.append(b); ss.append(s_)
        return torch.stack(cs), torch.stack(bs), torch.stack(ss)
    blk_full = pkg.fused_moe.MoeBlock(pack(2 * Fm, D, 1, 0, E, perm), pack(D, Fm, 2, 0, E), E, k, D, Fm)
    El = E // world
    blk_loc = pkg.fused_moe.MoeBlock(pack(2 * Fm, D, 1, rank * El, (rank + 1) * El, perm),
                                     pack(D, Fm, 2, rank * El, (rank + 1) * El), El, k, D, Fm)
    hm = torch.randn((L, D), generator=g, device="cuda").to(torch.bfloat16)
    lg = torch.randn((L, E), generator=g, device="cuda")
    lg[:, E - 3] = -30.0                                           # an expert nobody routes to
    refm = blk_full.step(hm, lg)
    Lr = L // world
    try:
        ep = P.PeerExpertParallelMoe(pkg, blk_loc, E, k, Lr)
    except Exception:   # noqa: BLE001
        ep = P.ExpertParallelMoe(pkg, blk_loc, E, k)
    sl = slice(rank * Lr, (rank + 1) * Lr)
    o1 = ep.step(hm[sl].contiguous(), lg[sl].contiguous())
    o2 = ep.step(hm[sl].contiguous(), lg[sl].contiguous())
    ok["ep"] = bool(torch.equal(o1, refm[sl])) and bool(torch.equal(o2, o1))
    torch.cuda.synchronize()
    pkg._lib.check_status()
    t = torch.tensor([int(ok["tp"]), int(ok["ep"])], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MIN)
    del tp, ep
    torch.cuda.empty_cache()
    return dict(tp=bool(t[0].item()), ep=bool(t[1].item()), world=world)


def gemm_only_roofline(pkg, torch, stack, pk, reps=3):
    """Average duration of the tcgen05 GEMM launches of one step, timed alone: every packed matrix is decoded to INT8
    beforehand (1.4 GB, far beyond L2), then the 112 GEMMs (with their real epilogues) are replayed back to back from a
    CUDA graph with events around the replay."""
    S = pkg.sc_kernels
    M = stack.M
    g = torch.Generator(device="cuda").manual_seed(7)
    wq = [{name: S.unpack_i8(c, b, n, k) for name, (c, b, _, n, k) in lw.items()} for lw in stack.layers]
    xq = {k: torch.randint(-127, 128, (M, k), dtype=torch.int8, device="cuda", generator=g) for k in (2048, 6144)}
    xs = torch.full((M,), 1e-2, device="cuda")
    res = torch.zeros((M, 2048), dtype=torch.bfloat16, device="cuda")

    def all_gemms():
        for lw, lq in zip(stack.layers, wq):
            for name, epi in (("qkv", 1), ("o", 2), ("gu", 3), ("down", 2)):
                _, _, ws, n, k = lw[name]
                S.mm_epi(xq[k], lq[name], xs, ws, epi, res=res if epi == 2 else None)
    all_gemms()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        all_gemms()
    for _ in range(2):
        graph.replay()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / reps
    n_launch = 4 * len(stack.layers)
    ops = qwen_ops(M, len(stack.layers))
    peak = 2 * pk["bf16_tflops"]          # the replay lasts ~10 ms at full clock: the burst figure applies
    ach = ops / ms / 1e9
    return dict(kernel="gemm_i8_kernel (tcgen05 kind::i8)", bound="tensor", achieved=ach, peak=peak, unit="TOP/s", frac=ach / peak,
                frac_of_nominal_4500=ach / 4500.0, traffic=NCU_GATEUP["dram_bytes"], launches=n_launch,
                avg_launch_us=ms * 1e3 / n_launch, algorithmic_ops_per_launch=ops / n_launch,
                peak_note=f"2 x bf16_tflops (burst) of {pk['source']} peaks: the file has no INT8 figure and the dense INT8 rate "
                          "is twice bf16",
                traffic_note=NCU_GATEUP["what"])


# DRAM traffic of the dominant launch as one ncu capture recorded it (dram__bytes_read.sum + dram__bytes_write.sum); bench.py
# cannot run the profiler itself, so the figure is carried here with what it was measured on.
NCU_GATEUP = dict(dram_bytes=29.5e6 + 0.12e6,
                  what="ncu --set full capture of one gate|up launch (2048 x 12288 x 2048, SwiGLU epilogue, `--case gemm`); "
                       "algorithmic operand bytes of that launch: 29.4 MB")


def run_ours(args):
    import torch
    import torch.distributed as dist
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    assert torch.cuda.is_available(), "bench.py needs a CUDA device (there is no CPU fallback)"
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    pkg = importlib.import_module("mxfp4-int8-m5_b200")
    if args.no_pdl:
        pkg._lib.call("scmx_set_pdl", 0)
    pk = peaks()
    if args.workload == "moe5":
        r = bench_moe5(pkg, torch, dist if world > 1 else None)
        if rank == 0:
            print(json.dumps(dict(metric="moe_prefill_tokens_per_s", value=r["tokens_per_s_one_layer"], unit="tokens/s (one layer)",
                                  n_gpus=world, config=dict(workload="large-MoE stress: 128 experts, F=768, block-16 format, "
                                                                     "Zipf(1.2) routing, 8192 tokens"), moe5=r)))
        if world > 1:
            dist.destroy_process_group()
        return
    parity = None
    if world > 1:
        try:
            parity = parity_multi(pkg, torch, dist)
        except Exception as e:   # noqa: BLE001
            parity = dict(tp=False, ep=False, error=f"{type(e).__name__}: {e}"[:200])
    M, layers, hidden = QWEN["M"], QWEN["layers"], 2048
    lw = build_dense_layers(pkg, torch, layers, shard=(rank, world))
    g = torch.Generator(device="cuda").manual_seed(123)
    h0 = torch.randn((M, hidden), generator=g, device="cuda").to(torch.bfloat16)
    o0 = torch.randn((M, hidden), generator=g, device="cuda").to(torch.bfloat16)
    collectives = "none"
    if world == 1:
        stack = pkg.fused_dense.DenseStack(lw, M, hidden, overlap=not args.no_overlap)
        hin, oin = h0, o0
    else:      # residual stream in segment layout [G, M, hidden/G]; this rank's columns of the attention output
        try:      # all-gathers as kernels over peer memory: the step can be replayed from a CUDA graph
            stack = pkg.parallel.PeerTensorParallelDense(pkg, lw, M, hidden, QWEN["groups"]["down"][1])
            collectives = "store-based all-gather kernels over NVLink peer memory"
        except Exception as e:   # noqa: BLE001
            print(f"# peer-memory path unavailable ({type(e).__name__}: {e}); using NCCL all-gather, eager launches", file=sys.stderr)
            stack = pkg.parallel.TensorParallelDense(pkg, lw, M, hidden)
            collectives = "NCCL all-gather"
        w = hidden // world
        hin = h0.view(M, world, w).permute(1, 0, 2).contiguous()
        oin = o0[:, rank * w:(rank + 1) * w].contiguous()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- warm-up (eager), then capture the step in a CUDA graph: ~340 launches per step are launch-bound from Python
    out = stack.step(hin, oin)
    torch.cuda.synchronize()
    pkg._lib.check_status()
    graph = None
    # (a multi-rank step with NCCL collectives is timed as eager launches; with peer-memory kernels it is captured)
    if not args.no_graph and (world == 1 or collectives.startswith("store")):
        try:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                out = stack.step(hin, oin)
        except Exception as e:   # noqa: BLE001
            print(f"# CUDA graph capture unavailable ({type(e).__name__}: {e}); timing eager launches", file=sys.stderr)
            graph = None
            torch.cuda.synchronize()
    run = graph.replay if graph is not None else (lambda: stack.step(hin, oin))
    for _ in range(max(args.warmup, 3)):
        run()
    barrier()
    # ---- timed: K steps, CUDA events on the launching stream, max over ranks.  The 718 MB of packed weights exceed L2
    # (126 MB), so every step streams its weights from HBM (no explicit flush needed).
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local) as cs:
        for _ in range(2):                   # the sampler's start-up left the GPU idle for a moment: two more untimed steps
            run()
        barrier()
        e0.record()
        for _ in range(args.steps):
            run()
        e1.record()
        barrier()
    clocks = cs.summary()

    def max_ms(ms):
        if world > 1:
            t = torch.tensor([ms], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return float(t.item())
        return ms
    ms = max_ms(e0.elapsed_time(e1) / args.steps)
    pkg._lib.check_status()
    ops = qwen_ops()
    value = ops / ms / 1e9

    # ---- e2e: the step's inputs come from pinned host memory and its result goes back to the host, every step
    hp, op_ = hin.cpu().pin_memory(), oin.cpu().pin_memory()
    outp = torch.empty_like(out, device="cpu").pin_memory()

    # Every step copies its inputs from pinned host memory and its result back.  The copies run on their own streams
    # through device-side staging buffers, so the transfers of step i + 1 / i - 1 overlap the compute of step i (PCIe is
    # full duplex); the main stream only does two device-to-device copies per step around the graph.
    main = torch.cuda.current_stream()
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    hin_s, oin_s, out_s = torch.empty_like(hin), torch.empty_like(oin), torch.empty_like(out)
    ev_in, ev_in_free, ev_out, ev_out_free = (torch.cuda.Event() for _ in range(4))

    def fetch_inputs():                       # host -> staging, once the previous contents were consumed
        with torch.cuda.stream(s_in):
            s_in.wait_event(ev_in_free)
            hin_s.copy_(hp, non_blocking=True)
            oin_s.copy_(op_, non_blocking=True)
            ev_in.record(s_in)

    def e2e_step():
        main.wait_event(ev_in)
        hin.copy_(hin_s, non_blocking=True)
        oin.copy_(oin_s, non_blocking=True)
        ev_in_free.record(main)
        fetch_inputs()                        # the next step's inputs travel while this step computes
        res = out
        if graph is not None:
            graph.replay()
        else:
            res = stack.step(hin, oin)
        main.wait_event(ev_out_free)          # the previous result has left the staging buffer
        out_s.copy_(res, non_blocking=True)
        ev_out.record(main)
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev_out)
            outp.copy_(out_s, non_blocking=True)
            ev_out_free.record(s_out)

    ev_in_free.record(main)
    ev_out_free.record(main)
    fetch_inputs()
    for _ in range(2):
        e2e_step()
    main.wait_stream(s_out)
    barrier()
    e0.record()
    for _ in range(args.steps):
        e2e_step()
    main.wait_stream(s_out)                   # the last result is on the host before the clock stops
    main.wait_stream(s_in)
    e1.record()
    barrier()
    ms_e2e = max_ms(e0.elapsed_time(e1) / args.steps)
    e2e = dict(value=ops / ms_e2e / 1e9, unit="TOPS", h2d_bytes_per_step=hp.numel() * 2 + op_.numel() * 2,
               d2h_bytes_per_step=outp.numel() * 2, ms_per_step=ms_e2e)

    line = dict(metric="w4a8_gemm_tops", value=value, unit="TOPS", n_gpus=world, steps=args.steps, warmup=max(args.warmup, 3),
                ms_per_step=ms, higher_is_better=True, scaling="strong", vs_baseline=None, dtype="int8", data="synthetic",
                config=dict(workload="qwen3-1.7b-shaped dense prefill: 28 layers x (qkv, o, gate|up, down), M=2048 tokens, "
                                     "SC-MXFP4 W4A8, random-init N(0,0.02) weights",
                            parallelism="single GPU" if world == 1 else f"tp{world}: weights sharded by output column, "
                                        f"4 all-gathers per layer ({collectives})",
                            l2="inputs larger than L2: 718 MB of packed weights per step", cuda_graph=graph is not None),
                clocks=clocks, e2e=e2e, gpu_launches=stack.launches_per_layer * layers * args.steps)
    if parity is not None:
        line["parity_multi"] = parity
    if args.dense_only:
        if rank == 0:
            print(json.dumps(line))
        return
    if world == 1:
        line["roofline"] = gemm_only_roofline(pkg, torch, stack, pk)
        line["decode"] = bench_decode(pkg, torch, stack, pk)
    del stack, lw, graph
    torch.cuda.empty_cache()
    try:
        line["moe"] = bench_moe(pkg, torch, dist if world > 1 else None)
    except Exception as e:   # noqa: BLE001
        line["moe"] = dict(error=f"{type(e).__name__}: {e}")
    if world > 1:
        torch.cuda.empty_cache()
        try:       # the same half-block with 4096 tokens per GPU (weak scaling of the expert-parallel path)
            line["moe_weak"] = bench_moe(pkg, torch, dist, weak=True)
        except Exception as e:   # noqa: BLE001
            line["moe_weak"] = dict(error=f"{type(e).__name__}: {e}")
    torch.cuda.empty_cache()
    try:
        line["moe5"] = bench_moe5(pkg, torch, dist if world > 1 else None)
    except Exception as e:   # noqa: BLE001
        line["moe5"] = dict(error=f"{type(e).__name__}: {e}"[:300])
    if world == 1:
        torch.cuda.empty_cache()
        try:       # whole-model time to first token and decode tokens/s through the fused callers (attention included)
            line["models"] = bench_models(pkg, torch, reps=3, lengths=(512, 2048))
        except Exception as e:   # noqa: BLE001
            line["models"] = dict(error=f"{type(e).__name__}: {e}")
    if rank == 0 and world == 1:
        threads = blas_threads()
        dt, cops = cpu_dense_layer_sample()
        line["cpu_baseline"] = dict(value=cops / dt / 1e12, unit="TOPS", cores=threads, kind="port",
                                    sample="1 of 28 layers at M=2048: act-quant + f64-BLAS INT32 GEMM + epilogue (NumPy oracle)")
        gdt, gbytes = cpu_gemv_sample()
        line["cpu_baseline"]["gemv"] = dict(value=gbytes / gdt / 1e9, unit="GB/s (of 4-bit packed bytes)", cores=1,
                                            us_per_gemv=gdt / 4 * 1e6,
                                            sample="the 4 GEMVs of one layer: int64 matrix-vector product (NumPy, no BLAS) + epilogue")
        mdt, mtok = cpu_moe_sample()
        line["cpu_baseline"]["moe"] = dict(value=mtok / mdt, unit="tokens/s (one half-block)", cores=threads,
                                           sample=f"{mtok} tokens (4096 sorted rows): act-quant, per-expert f64-BLAS loop for "
                                                  "gate|up + SwiGLU, act-quant, per-expert loop for down")
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def bench_models(pkg, torch, reps=5, lengths=(512, 2048, 8192), kinds=("qwen3", "olmoe")):
    """Whole-model numbers through the fused callers (attention, KV cache and the output head included): time to first
    token = prefill + the last position's logits, and batch-1 decode tokens/s, for synthetic-weight models of the two
    architectures, next to the same torch model in bf16 (unfused, torch's GEMMs)."""
    HM, FQ, FO, DEC = pkg.host_model, pkg.fused_qwen3, pkg.fused_olmoe, pkg.decode
    out = {}

    def timed(fn, n):
        for _ in range(2):
            fn()
        torch.cuda.synchronize()
        ts = []
        for _ in range(n):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        return float(np.median(ts))

    for kind in kinds:
        a = HM.QWEN3_1_7B if kind == "qwen3" else HM.OLMOE_1B_7B
        with torch.device("cuda"):
            model = HM.CausalLM(a)
        model.init_random(seed=0, scale=0.02)
        res = {"params_b": round(sum(p.numel() for p in model.parameters()) / 1e9, 2)}
        ids_all = torch.randint(0, a.vocab_size, (1, max(lengths) + 64), device="cuda")
        cap = max(lengths) + 64

        def bf16_prefill(L):
            cache = HM.make_prompt_cache(model, cap)
            h = model.model.embed_tokens(ids_all[:, :L])[0]
            for layer, c in zip(model.model.layers, cache):
                h = layer(h, c)
            return model.head(model.model.norm(h[-1:])[None])

        with torch.no_grad():
            if kind == "qwen3":          # the loop over experts of the unfused MoE block is not a fair bf16 baseline
                res["bf16_ttft_ms"] = {str(L): round(timed(lambda: bf16_prefill(L), reps), 3) for L in lengths}
        fused = (FQ.FusedQwen3(model, FQ.pack_model(model, on_device=True)) if kind == "qwen3"
                 else FO.FusedOlmoe(model, FO.pack_olmoe(model, on_device=True)))
        res["packed_gb"] = round(fused.weight_bytes() / 1e9, 3)
        cache = fused.make_cache(cap)

        def prefill(L):
            for c in cache:
                c.offset = 0
            return fused.logits(fused.hidden(ids_all[:, :L], cache)[:, -1:])

        res["ttft_ms"], res["ttft_graph_ms"] = {}, {}
        for L in lengths:
            res["ttft_ms"][str(L)] = round(timed(lambda: prefill(L), reps), 3)
            try:
                g = torch.cuda.CUDAGraph()
                s = torch.cuda.Stream()
                s.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(s):
                    prefill(L)
                    torch.cuda.synchronize()
                    with torch.cuda.graph(g, stream=s):
                        prefill(L)
                torch.cuda.current_stream().wait_stream(s)
                res["ttft_graph_ms"][str(L)] = round(timed(g.replay, reps), 3)
                del g
            except Exception as e:  # noqa: BLE001
                res["ttft_graph_ms"][str(L)] = f"capture failed: {str(e)[:80]}"
        # decode: 64 tokens after a 512-token prompt.  Graph-replayed steps with (dense) the persistent one-kernel step and
        # with the chain of stand-alone kernels, and eager step() calls
        cls = DEC.DecodeQwen3 if kind == "qwen3" else DEC.DecodeOlmoe
        n_tok = 64
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

        def tok_s(fn):
            for rep in range(2):                               # first pass warms up (and captures), second is timed
                prefill(512)
                e0.record()
                fn()
                e1.record()
                torch.cuda.synchronize()
            return round(n_tok / (e0.elapsed_time(e1) / 1e3), 1)

        def eager(dec):
            tok = ids_all[:, 512:513]
            for _ in range(n_tok):
                tok = dec.step(tok, cache)[:, -1].argmax(-1, keepdim=True)

        dec = cls(fused)
        res["decode_tok_s"] = tok_s(lambda: dec.generate(ids_all[:, 512:513], cache, n_tok))
        res["decode_tok_s_eager"] = tok_s(lambda: eager(dec))
        if kind == "qwen3":
            res["decode_persistent_kernel"] = bool(dec.persistent)
            dec.check_status()
            chain = cls(fused, persistent=False)
            res["decode_tok_s_kernel_chain"] = tok_s(lambda: chain.generate(ids_all[:, 512:513], cache, n_tok))
            del chain
        pkg._lib.check_status()
        out[kind] = res
        del fused, dec, cache, model
        torch.cuda.empty_cache()
    return out


def run_case(args):
    """Small single-kernel cases for profiler captures (a few launches, a few hundred MB at most)."""
    import torch
    torch.cuda.set_device(0)
    pkg = importlib.import_module("mxfp4-int8-m5_b200")
    S, G, F = pkg.sc_kernels, pkg.sc_decode, pkg.sc_format
    g = torch.Generator(device="cuda").manual_seed(0)
    if args.case == "gemm":       # the gate|up GEMM of one layer: 2048 x 12288 x 2048, SwiGLU epilogue
        xq = torch.randint(-127, 128, (2048, 2048), dtype=torch.int8, device="cuda", generator=g)
        wq = torch.randint(-96, 97, (12288, 2048), dtype=torch.int8, device="cuda", generator=g)
        xs = torch.full((2048,), 1e-2, device="cuda")
        ws = torch.full((12288,), 2.0 ** -9, device="cuda")
        for _ in range(4):
            S.mm_epi(xq, wq, xs, ws, 3)
    elif args.case == "gemmw4":   # the same GEMM straight from packed weights (tiles expanded inside the K loop)
        xq = torch.randint(-127, 128, (2048, 2048), dtype=torch.int8, device="cuda", generator=g)
        w = torch.randn((12288, 2048), generator=g, device="cuda") * 0.02
        c, b, ws, _, _ = F.quantize_device(w, want_qw=False)
        xs = torch.full((2048,), 1e-2, device="cuda")
        for _ in range(4):
            S.mm_w4_epi(xq, c, b, xs, ws, 12288, 3)
    elif args.case == "gemmlib":  # this repository's INT8 GEMM beside the library's (torch._int_mm = cuBLASLt) on the same operands
        def per_launch(fn, n):
            for _ in range(3):
                fn()
            gr = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gr):
                for _ in range(n):
                    fn()
            for _ in range(2):
                gr.replay()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            e0.record()
            for _ in range(5):
                gr.replay()
            e1.record()
            torch.cuda.synchronize()
            return e0.elapsed_time(e1) / 5 / n * 1e3
        rows = []
        for (M, N, K) in [(2048, 4096, 2048), (2048, 2048, 2048), (2048, 12288, 2048), (2048, 2048, 6144), (8192, 8192, 8192), (4096, 14336, 4096)]:
            xq = torch.randint(-127, 128, (M, K), dtype=torch.int8, device="cuda", generator=g)
            wq = torch.randint(-96, 97, (N, K), dtype=torch.int8, device="cuda", generator=g)
            xs = torch.rand(M, device="cuda", generator=g) * 1e-3
            ws = torch.rand(N, device="cuda", generator=g) * 1e-3
            wt = wq.t()
            n = 4 if M >= 4096 else 10
            same = bool(torch.equal(S.mm_i8_i32(xq, wq)[:M], torch._int_mm(xq, wt)))
            ops = 2 * M * N * K
            t = dict(int32=per_launch(lambda: S.mm_i8_i32(xq, wq), n), bf16_epilogue=per_launch(lambda: S.mm_epi(xq, wq, xs, ws, 1), n),
                     library_int32=per_launch(lambda: torch._int_mm(xq, wt), n))
            rows.append(dict(shape=[M, N, K], equal_int32=same, us=t, tops={k: ops / v / 1e6 for k, v in t.items()}))
        print(json.dumps(dict(case="gemmlib", rows=rows)))
        return
    elif args.case == "rows":     # the row kernels between the GEMMs of a dense layer at M = 2048: RMSNorm + INT8 and act-quant
        h = torch.randn((2048, 2048), generator=g, device="cuda").to(torch.bfloat16)
        act = torch.randn((2048, 6144), generator=g, device="cuda").to(torch.bfloat16)
        nw = torch.ones(2048, dtype=torch.bfloat16, device="cuda")
        for _ in range(3):
            S.rmsnorm_quant(h, nw, 1e-6, 2048)
            S.act_quant(h, 2048)
            S.act_quant(act, 2048)
    elif args.case == "gemv":     # 12 distinct gate|up weight sets (154 MB > L2), one GEMV each, two passes
        sets = []
        for _ in range(12):
            w = torch.randn((12288, 2048), generator=g, device="cuda") * 0.02
            sets.append(F.quantize_device(w, want_qw=False)[:3])
        xq = torch.randint(-127, 128, (2048,), dtype=torch.int8, device="cuda", generator=g)
        xs = torch.full((1,), 1e-2, device="cuda")
        for _ in range(2):
            for c, b, w_ in sets:
                G.gemv(xq, c, b, xs, w_, 12288, 3)
    elif args.case == "gemvlist":  # 24 GEMVs (6 layers x qkv, o, gate|up, down; 154 MB of packed weights) as one persistent launch, 3 launches
        jobs = []
        xqs = {k: torch.randint(-127, 128, (k,), dtype=torch.int8, device="cuda", generator=g) for k in (2048, 6144)}
        xs = torch.full((1,), 1e-2, device="cuda")
        res = torch.zeros(2048, dtype=torch.bfloat16, device="cuda")
        for _ in range(6):
            for (n, k), epi in zip(QWEN["groups"].values(), (1, 2, 3, 2)):
                c, b, w_, _, _ = F.quantize_device(torch.randn((n, k), generator=g, device="cuda") * 0.02, want_qw=False)
                jobs.append((xqs[k], c, b, xs, w_, n, epi, res if epi == 2 else None))
        gl = G.GemvList(jobs)
        for _ in range(3):
            gl.run()
    elif args.case == "gemvbig":  # one LM-head-shaped GEMV, 151936 x 2048 (160 MB of packed weights), three launches
        w = torch.randn((151936, 2048), generator=g, device="cuda") * 0.02
        c, b, w_, _, _ = F.quantize_device(w, want_qw=False)
        del w
        xq = torch.randint(-127, 128, (2048,), dtype=torch.int8, device="cuda", generator=g)
        xs = torch.full((1,), 1e-2, device="cuda")
        for _ in range(3):
            G.gemv(xq, c, b, xs, w_, 151936, 1)
    elif args.case in ("decodestep", "decodechain"):   # Qwen3-1.7B-shaped model, 512 positions in the cache: three one-kernel
        # decode steps, or two graph-replayed steps of the chain of stand-alone kernels
        HM, FQ, DEC = pkg.host_model, pkg.fused_qwen3, pkg.decode
        with torch.device("cuda"):
            model = HM.CausalLM(HM.QWEN3_1_7B)
        model.init_random(0)
        fused = FQ.FusedQwen3(model, FQ.pack_model(model, on_device=True))
        dec = DEC.DecodeQwen3(fused, persistent=args.case == "decodestep")
        ids = torch.randint(0, HM.QWEN3_1_7B.vocab_size, (1, 513), device="cuda", generator=g)
        cache = fused.make_cache(1024)
        fused.logits(fused.hidden(ids[:, :512], cache)[:, -1:])
        tok = ids[:, 512:513]
        if args.case == "decodestep":
            for _ in range(3):
                tok = dec.step(tok, cache)[:, -1].argmax(-1, keepdim=True)
        else:       # the chain of stand-alone kernels: capture the step, then replay two tokens inside the profiler range
            dec.generate(tok, cache, 1)
            torch.cuda.synchronize()
            torch.cuda.profiler.start()
            dec.generate(tok, cache, 2)
            torch.cuda.synchronize()
            torch.cuda.profiler.stop()
        torch.cuda.synchronize()
        dec.check_status()
    elif args.case == "ep1":      # the per-rank work of the 8-GPU expert-parallel half-block on one GPU: a world of one rank
        # with 8 experts (top-8: every token visits all of them) and 512 tokens = 4096 rows, through the peer-memory kernels
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29533")
        dist.init_process_group("nccl", rank=0, world_size=1, device_id=torch.device("cuda", 0))
        cfg = dict(OLMOE, E=8, tokens=512)
        blk = build_moe_block(pkg, torch, cfg=cfg, shard=(0, 1))
        blk.early = False
        layer = pkg.parallel.PeerExpertParallelMoe(pkg, blk, 8, 8, 512)
        h = torch.randn((512, 2048), generator=g, device="cuda").to(torch.bfloat16)
        lg = torch.randn((512, 8), generator=g, device="cuda")
        for _ in range(3):
            layer.step(h, lg)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            layer.step(h, lg)
        for _ in range(3):
            graph.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(20):
            graph.replay()
        e1.record()
        torch.cuda.synchronize()
        print(json.dumps(dict(case="ep1", ms_per_half_block=e0.elapsed_time(e1) / 20)))
        torch.cuda.profiler.start()
        graph.replay()
        torch.cuda.synchronize()
        torch.cuda.profiler.stop()
        pkg._lib.check_status()
        dist.destroy_process_group()
        return
    elif args.case == "models":
        print(json.dumps(dict(case="models", models=bench_models(pkg, torch))))
        return
    elif args.case == "moe512":   # the half-block at 512 tokens: 64 rows per expert, the grouped GEMMs read the packed weights
        bench_moe(pkg, torch, None, reps=1, tokens=512)
    else:
        bench_moe(pkg, torch, None, reps=1)
    torch.cuda.synchronize()
    pkg._lib.check_status()
    print(json.dumps(dict(case=args.case, ok=True)))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--no-overlap", action="store_true", help="decode weights on the main stream instead of a side stream")
    ap.add_argument("--no-pdl", action="store_true", help="launch without programmatic stream serialization")
    ap.add_argument("--dense-only", action="store_true", help="skip the roofline / decode / MoE / CPU sections")
    ap.add_argument("--workload", default="all", choices=["all", "moe5"], help="moe5: only the large-MoE stress section")
    ap.add_argument("--case", choices=["gemm", "gemmw4", "gemmlib", "rows", "gemv", "gemvbig", "gemvlist", "moe", "moe512", "ep1", "models", "decodestep", "decodechain"], help="run one small kernel case (for profiler captures) and exit")
    args = ap.parse_args()
    if args.case:
        run_case(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
