"""Grouped SC-MXFP4 W4A8 expert GEMM for mixture-of-experts prefill, with the call signatures of the reference's
e2e/sc_moe.py (route_sort, segments, moe_mm, moe_mm_i8, unpack_experts) plus the combine kernel of
e2e/fused_olmoe.py (moe_combine) and on-device routing (router_topk, gather_rows).

Token-expert assignments are sorted by expert so that expert e owns rows [off[e], off[e+1]) of the gathered INT8
activations; one persistent tcgen05 kernel covers all experts, finding the expert and M tile of each slot from
`tstart`.  The M tile is 128 rows: pass tm = 128 to route_sort / segments.
"""
import torch

from . import _lib
from . import sc_format as F
from . import sc_kernels as S

TM = 128
EXPERTS_PER_PASS = 32    # experts decoded to INT8 per pass of moe_mm (two rotating scratch halves); 8 -> 32: -12 % on the half-block

# moe_mm expands the packed expert tiles inside the GEMM kernel (scmx_moe_mm_w4) where the format allows it; False selects the
# older form that decodes groups of experts to an INT8 scratch between GEMM passes (scmx_moe_mm).
FUSED_UNPACK = True

_scratch = {}


def route_sort(inds, n_experts, tm=TM):
    """inds int [M, topk] -> (pos int32 [M*topk], tok int32 [M*topk + tm], e_sorted int32 [M*topk], off int32 [E+1],
    tstart int32 [E+1], max M-tiles)."""
    _lib.require_cuda(inds)
    M, k = inds.shape
    R = M * k
    inds = inds.to(torch.int32).contiguous()
    dev = inds.device
    pos = torch.empty(R, dtype=torch.int32, device=dev)
    tok = torch.empty(R + tm, dtype=torch.int32, device=dev)
    es = torch.empty(R, dtype=torch.int32, device=dev)
    off = torch.empty(n_experts + 1, dtype=torch.int32, device=dev)
    ts = torch.empty(n_experts + 1, dtype=torch.int32, device=dev)
    _lib.call("scmx_route_sort", _lib.ptr(inds), M, k, n_experts, tm, _lib.ptr(pos), _lib.ptr(tok), _lib.ptr(es),
              _lib.ptr(off), _lib.ptr(ts), _lib.stream())
    return pos, tok, es, off, ts, -(-R // tm) + n_experts


def segments(expert_sorted, n_experts, tm=TM):
    """Sorted expert id per row -> (off int32 [E+1], tstart int32 [E+1], max number of M-tiles)."""
    R = expert_sorted.shape[0]
    counts = torch.bincount(expert_sorted.to(torch.int64), minlength=n_experts).to(torch.int32)
    zero = torch.zeros(1, dtype=torch.int32, device=expert_sorted.device)
    off = torch.cat([zero, torch.cumsum(counts, 0).to(torch.int32)])
    tiles = (counts + tm - 1) // tm
    tstart = torch.cat([zero, torch.cumsum(tiles, 0).to(torch.int32)])
    return off, tstart, -(-R // tm) + n_experts


def router_topk(logits, k):
    """logits f32 [M, E] -> (inds int32 [M, k], scores bf16 [M, k]): softmax then top-k, scores not renormalised."""
    _lib.require_cuda(logits)
    M, E = logits.shape
    logits = logits.float().contiguous()
    inds = torch.empty((M, k), dtype=torch.int32, device=logits.device)
    scores = torch.empty((M, k), dtype=torch.bfloat16, device=logits.device)
    _lib.call("scmx_router_topk", _lib.ptr(logits), M, E, k, _lib.ptr(inds), _lib.ptr(scores), None, _lib.stream())
    return inds, scores


def gather_rows(xq, xs, tok, R):
    """(xq[tok], xs[tok[:R]]): INT8 rows and scales of the sorted assignments (tok has R + tm entries)."""
    _lib.require_cuda(xq, xs, tok)
    rows, K = tok.shape[0], xq.shape[1]
    dq = torch.empty((rows, K), dtype=torch.int8, device=xq.device)
    ds = torch.empty(R, dtype=torch.float32, device=xq.device)
    _lib.call("scmx_gather_rows", _lib.ptr(xq), _lib.ptr(xs), _lib.ptr(tok), rows, R, K, _lib.ptr(dq), _lib.ptr(ds),
              _lib.stream())
    return dq, ds


def _out(R, N, epi, dev):
    if epi == 0:
        return torch.empty((R, N), dtype=torch.int32, device=dev)
    return torch.empty((R, N // 2 if epi == 3 else N), dtype=torch.bfloat16, device=dev)


def moe_mm(xq, R, codes, bcodes, wscale, off, tstart, max_tiles, N, epi, xscale=None, dtype=torch.bfloat16,
           tile=(TM, 256, 4), bk=128):
    """xq int8 [>= R + TM, K]: R rows sorted by expert (+ padding rows, never stored); packed expert weights codes
    [E, N*K/8], bcodes [E, N, ...], wscale f32 [E, N] -> INT32 [R, N] (EPI 0), bf16 [R, N] (1) or bf16 [R, N/2] (3)."""
    _lib.require_cuda(xq, codes, bcodes, wscale, off, tstart, xscale)
    K = xq.shape[1]
    assert xq.shape[0] >= R + TM and epi in (0, 1, 3)
    E = wscale.shape[0]
    assert N % 32 == 0 and K % 16 == 0 and codes.numel() == E * N * K // 8
    out = _out(R, N, epi, xq.device)
    if FUSED_UNPACK and E <= 512 and _lib.lib().scmx_w4_supported(F.DEFAULT.c_struct(), K):
        _lib.call("scmx_moe_mm_w4", _lib.ptr(xq), R, _lib.ptr(codes), _lib.ptr(bcodes), _lib.ptr(wscale), _lib.ptr(off), E, N, K,
                  F.DEFAULT.c_struct(), epi, _lib.ptr(xscale), _lib.ptr(out), _lib.ptr(_lib.status_buffer()), _lib.stream())
        return out
    epp = min(EXPERTS_PER_PASS, E)
    need = 2 * epp * N * K
    key = (xq.device.index, need)
    if key not in _scratch:
        _scratch.clear()
        _scratch[key] = torch.empty(need + 1024, dtype=torch.int8, device=xq.device)
    buf = _scratch[key]
    base = (-buf.data_ptr()) % 1024
    _lib.call("scmx_moe_mm", _lib.ptr(xq), R, _lib.ptr(codes), _lib.ptr(bcodes), _lib.ptr(wscale), _lib.ptr(off),
              _lib.ptr(tstart), E, N, K, F.DEFAULT.c_struct(), epi, _lib.ptr(xscale), _lib.ptr(out), TM, epp,
              _lib.c_vp(buf.data_ptr() + base), need, _lib.ptr(_lib.status_buffer()), _lib.stream())
    return out


def moe_mm_i8(xq, R, wq, wscale, off, tstart, max_tiles, N, epi, xscale=None, dtype=torch.bfloat16, tile=(TM, 256, 4)):
    """Two-pass variant of moe_mm: wq int8 [E * N, K] already unpacked (unpack_experts)."""
    _lib.require_cuda(xq, wq, wscale, off, tstart, xscale)
    K = xq.shape[1]
    E = wscale.shape[0]
    assert xq.shape[0] >= R + TM and tuple(wq.shape) == (E * N, K) and epi in (0, 1, 3)
    out = _out(R, N, epi, xq.device)
    _lib.call("scmx_moe_mm_i8", _lib.ptr(xq), R, _lib.ptr(wq), _lib.ptr(wscale), _lib.ptr(off), _lib.ptr(tstart), E, N, K,
              epi, _lib.ptr(xscale), _lib.ptr(out), TM, _lib.ptr(_lib.status_buffer()), _lib.stream())
    return out


def unpack_experts(codes, bcodes, N, K):
    """All experts' packed weights -> INT8 [E * N, K] (one unpack launch)."""
    E = codes.shape[0]
    return S.unpack_i8(codes.reshape(-1), bcodes.reshape(E * N, -1), E * N, K)


def moe_combine(y, pos, scores, res, w, eps, M, quant=True):
    """y bf16 [R, K] (sorted assignments), pos int32 [M*topk], scores bf16 [M, topk], res bf16 [Mp, K] ->
    (h [Mp, K], xq int8 [Mp, K], xscale [Mp]) with xq = INT8(rms_norm(h, w)) when quant."""
    _lib.require_cuda(y, pos, scores, res, w)
    Mp, K = res.shape
    topk = scores.shape[1]
    assert y.dtype == torch.bfloat16 and scores.dtype == torch.bfloat16 and res.dtype == torch.bfloat16
    dev = res.device
    h = torch.empty((Mp, K), dtype=torch.bfloat16, device=dev)
    xq = torch.empty((Mp, K), dtype=torch.int8, device=dev)
    xs = torch.empty(Mp, dtype=torch.float32, device=dev)
    _lib.call("scmx_moe_combine", _lib.ptr(y), _lib.ptr(pos), _lib.ptr(scores), _lib.ptr(res), _lib.ptr(w),
              S._eps(eps), M, Mp, K, topk, int(bool(quant)), _lib.ptr(h), _lib.ptr(xq), _lib.ptr(xs), _lib.stream())
    return h, xq, xs
