"""Batch-1 decode GEMV that reads the packed SC-MXFP4 weights directly, with the call signature of the reference's
e2e/sc_decode.py `gemv`.  The kernel accumulates exact INT32 totals (DP4A) and applies the GEMM's epilogues, so
decode and prefill produce the same bits.  Prologues pro=1 / pro=2 (activation quantization / RMSNorm + quantization
of a bf16 input row) run as the separate row kernel followed by the GEMV, or - on request, see FUSE_PROLOGUE - inside the
GEMV kernel (scmx_gemv_pro; K <= 8192, register kernel only).  Both give the same bits."""
import ctypes

import torch

from . import _lib
from . import sc_format as F
from . import sc_kernels as S

USE_PDL = True   # programmatic dependent launch: weight loads overlap the previous kernel's tail
# Which prologues run inside the GEMV kernel (scmx_gemv_pro) where it applies.  Empty by default: in a chain of programmatic
# dependent launches the separate row kernel is faster (Qwen3-1.7B decode from a graph: 638 tokens/s with none fused, 628 /
# 625 / 605 with pro 1 / pro 2 / both fused), because every CTA of the GEMV repeats the row reductions.
FUSE_PROLOGUE = ()


def gemv(xq, codes, bcodes, xscale, wscale, N, epi, dtype=torch.bfloat16, res=None, nsg=None, eidx=None, xstride=0,
         pro=0, nw=None, eps=None, rows=None, vpl=None, shared=None, splitk=None, fuse=None):
    """W4A8 GEMV.  pro=0: xq int8 [K] (or [S, K] with xstride=1) and xscale; pro=1: xq is a bf16 row (or rows),
    quantized per token first; pro=2: RMSNorm(nw, eps) + INT8 first.  Output: EPI 1: bf16 [N]; 2: bf16 [N] = res + y;
    3: bf16 [N / 2] (interleaved gate/up rows); 0: int32 [N] exact totals.
    MoE (eidx int32 [S] given): codes [E, ...], bcodes [E, N, ...], wscale [E, N]; output row j uses expert eidx[j] and
    input row j if xstride = 1 (else the single input row) -> [S, N or N/2].  shared = e: one more slot uses expert e.
    nsg / rows / vpl / splitk are Metal tile hints: accepted and ignored.  fuse: None = FUSE_PROLOGUE, True / False / a tuple
    of prologue numbers = run them inside the GEMV kernel."""
    xbf = None
    if pro:
        x2 = xq.reshape(-1, xq.shape[-1])
        Kp = x2.shape[-1]
        sel = FUSE_PROLOGUE if fuse is None else fuse
        fused = (pro in (sel if isinstance(sel, tuple) else ((1, 2) if sel else ())) and epi != 0 and Kp <= 8192 and x2.dtype == torch.bfloat16 and x2.is_contiguous()
                 and (eidx is not None or N * Kp // 2 < (16 << 20)))
        if fused:
            xbf = x2
        else:
            xq, xscale = (S.act_quant(x2, x2.shape[0]) if pro == 1 else S.rmsnorm_quant(x2, nw, eps, x2.shape[0]))
    _lib.require_cuda(xq, codes, bcodes, xscale, wscale, res, eidx)
    K = xq.shape[-1]
    nslot = 0 if eidx is None else eidx.numel()
    S_ = 1 if eidx is None else nslot + (shared is not None)
    assert K % 128 == 0 and N % 4 == 0 and epi in (0, 1, 2, 3)
    assert dtype == torch.bfloat16
    no = N // 2 if epi == 3 else N
    out = torch.empty(S_ * no, dtype=torch.int32 if epi == 0 else torch.bfloat16, device=xq.device)
    if eidx is not None:
        eidx = eidx.to(torch.int32)
    if xbf is not None:
        _lib.require_cuda(nw)
        _lib.call("scmx_gemv_pro", _lib.ptr(xbf), pro, _lib.ptr(nw) if pro == 2 else None, S._eps(eps) if pro == 2 else 0.0,
                  _lib.ptr(codes), _lib.ptr(bcodes), _lib.ptr(wscale), N, K, F.DEFAULT.c_struct(), epi,
                  _lib.ptr(res) if epi == 2 else None, _lib.ptr(eidx), nslot, -1 if shared is None else int(shared), xstride,
                  _lib.ptr(out), int(USE_PDL), _lib.stream())
    else:
        _lib.call("scmx_gemv", _lib.ptr(xq), _lib.ptr(xscale), _lib.ptr(codes), _lib.ptr(bcodes), _lib.ptr(wscale), N, K,
                  F.DEFAULT.c_struct(), epi, _lib.ptr(res) if epi == 2 else None, _lib.ptr(eidx), nslot,
                  -1 if shared is None else int(shared), xstride, _lib.ptr(out), int(USE_PDL), _lib.stream())
    return out if eidx is None else out.reshape(S_, no)


class GemvList:
    """A list of independent dense GEMVs run as ONE persistent launch (scmx_gemv_multi): the packed weights of all jobs
    stream through one shared-memory ring without a pause at matrix boundaries.  jobs: iterable of
    (xq int8 [K], codes, bcodes, xscale f32 [1], wscale, N, epi, res-or-None); every input must be complete before run()
    is launched (jobs cannot feed each other).  Outputs are allocated once and reused by every run()."""

    def __init__(self, jobs):
        jobs = list(jobs)
        assert 1 <= len(jobs) <= 512
        self.n = len(jobs)
        self.keep = jobs                                  # the tensors the records point at
        self.fmt = F.DEFAULT
        self.host = (_lib.ScmxGemvJob * self.n)()
        self.outs = []
        for rec, (xq, codes, bcodes, xscale, wscale, N, epi, res) in zip(self.host, jobs):
            _lib.require_cuda(xq, codes, bcodes, xscale, wscale, res)
            assert xq.dtype == torch.int8 and xq.dim() == 1 and epi in (0, 1, 2, 3)
            no = N // 2 if epi == 3 else N
            out = torch.empty(no, dtype=torch.int32 if epi == 0 else torch.bfloat16, device=xq.device)
            self.outs.append(out)
            rec.codes, rec.bcodes, rec.wscale, rec.xq = codes.data_ptr(), bcodes.data_ptr(), wscale.data_ptr(), xq.data_ptr()
            rec.xscale = xscale.data_ptr() if xscale is not None else None
            rec.res = res.data_ptr() if (epi == 2 and res is not None) else None
            rec.out, rec.N, rec.K, rec.epi = out.data_ptr(), N, xq.shape[0], epi
        _lib.call("scmx_gemv_multi_plan", ctypes.byref(self.host), self.n, self.fmt.c_struct())
        raw = torch.frombuffer(bytearray(bytes(self.host)), dtype=torch.uint8).clone()
        self.dev = raw.to(jobs[0][0].device)
        self.tiles = int(self.host[0].plan[8])

    def run(self):
        _lib.call("scmx_gemv_multi", ctypes.byref(self.host), _lib.ptr(self.dev), self.n, self.fmt.c_struct(),
                  _lib.ptr(_lib.status_buffer()), int(USE_PDL), _lib.stream())
        return self.outs
