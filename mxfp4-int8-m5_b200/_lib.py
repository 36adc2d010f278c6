"""ctypes binding of libscmx.so, the C-ABI library that holds every CUDA kernel of this package.

There is no CPU fallback: if the library is missing, or a call fails, an exception is raised.
"""
import ctypes
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libscmx.so")

c_i64, c_int, c_float, c_vp = ctypes.c_int64, ctypes.c_int, ctypes.c_float, ctypes.c_void_p


class ScmxFormat(ctypes.Structure):
    """Mirror of `scmx_format` in include/scmx.h."""
    _fields_ = [("block", ctypes.c_int32), ("bc_bits", ctypes.c_int32), ("n_mult", ctypes.c_int32),
                ("code_mag", ctypes.c_int32 * 8), ("mult", ctypes.c_int32 * 16)]


class ScmxDecodeLayer(ctypes.Structure):
    """Mirror of `scmx_decode_layer` in include/scmx.h."""
    _fields_ = [("codes", ctypes.c_void_p * 4), ("bcodes", ctypes.c_void_p * 4), ("wscale", ctypes.c_void_p * 4),
                ("ln_in", ctypes.c_void_p), ("ln_post", ctypes.c_void_p), ("q_norm", ctypes.c_void_p),
                ("k_norm", ctypes.c_void_p), ("k_cache", ctypes.c_void_p), ("v_cache", ctypes.c_void_p)]


class ScmxGemvJob(ctypes.Structure):
    """Mirror of `scmx_gemv_job` in include/scmx.h (128 bytes)."""
    _fields_ = [("codes", ctypes.c_void_p), ("bcodes", ctypes.c_void_p), ("wscale", ctypes.c_void_p), ("xq", ctypes.c_void_p),
                ("xscale", ctypes.c_void_p), ("res", ctypes.c_void_p), ("out", ctypes.c_void_p), ("N", ctypes.c_int32),
                ("K", ctypes.c_int32), ("epi", ctypes.c_int32), ("plan", ctypes.c_int32 * 15)]


class ScmxError(RuntimeError):
    """A libscmx entry point returned a non-zero status."""


_FMT_P = ctypes.POINTER(ScmxFormat)
# name -> argument types (every entry point returns int unless listed in _RESTYPE)
SIGNATURES = {
    "scmx_abi_version": [],
    "scmx_last_error_string": [],
    "scmx_quantize_sc_mxfp4": [c_vp, c_int, c_i64, c_i64, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp],
    "scmx_quantize_family": [c_vp, c_i64, c_i64, _FMT_P, c_int, c_vp, c_vp, c_vp, c_vp, c_vp],
    "scmx_unpack_i8": [c_vp, c_vp, c_i64, c_i64, _FMT_P, c_vp, c_vp],
    "scmx_act_quant": [c_vp, c_i64, c_i64, c_i64, c_vp, c_vp, c_vp],
    "scmx_rmsnorm_quant": [c_vp, c_vp, c_float, c_i64, c_i64, c_i64, c_vp, c_vp, c_vp, c_vp],
    "scmx_act_quant_seg": [c_vp, c_i64, c_i64, c_i64, c_int, c_i64, c_vp, c_vp, c_vp],
    "scmx_rmsnorm_quant_seg": [c_vp, c_vp, c_float, c_i64, c_i64, c_i64, c_int, c_i64, c_vp, c_vp, c_vp, c_vp],
    "scmx_res_epilogue": [c_vp, c_vp, c_vp, c_vp, c_i64, c_i64, c_vp, c_vp],
    "scmx_swiglu_quant": [c_vp, c_vp, c_vp, c_i64, c_i64, c_vp, c_vp, c_vp],
    "scmx_swiglu": [c_vp, c_vp, c_i64, c_vp, c_vp],
    "scmx_rot_quant": [c_vp, c_vp, c_i64, c_i64, c_i64, c_vp, c_vp, c_vp],
    "scmx_qkv_norm": [c_vp, c_int, c_vp, c_vp, c_vp, c_vp, c_float, c_i64, c_int, c_int, c_int, c_int, c_vp, c_vp, c_i64, c_i64, c_vp, c_vp,
                      c_i64, c_vp, c_vp, c_i64, c_i64, c_vp],
    "scmx_attn_decode": [c_vp, c_vp, c_vp, c_i64, c_vp, c_i64, c_float, c_int, c_int, c_int, c_int, c_vp, c_vp, c_vp, c_vp],
    "scmx_mm_i8": [c_vp, c_vp, c_i64, c_i64, c_i64, c_int, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp],
    "scmx_w4_supported": [_FMT_P, c_i64],
    "scmx_mm_w4": [c_vp, c_vp, c_vp, c_i64, c_i64, c_i64, _FMT_P, c_int, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp],
    "scmx_moe_mm_w4": [c_vp, c_i64, c_vp, c_vp, c_vp, c_vp, c_int, c_i64, c_i64, _FMT_P, c_int, c_vp, c_vp, c_vp, c_vp],
    "scmx_moe_mm_w4_ret": [c_vp, c_i64, c_vp, c_vp, c_vp, c_vp, c_int, c_i64, c_i64, _FMT_P, c_vp, c_vp, c_vp, c_int, c_vp, c_vp,
                           c_vp],
    "scmx_mm_i8_bcast": [c_vp, c_vp, c_i64, c_i64, c_i64, c_int, c_vp, c_vp, c_vp, c_vp, c_int, c_vp, c_vp],
    "scmx_set_gemm_tile": [c_int],
    "scmx_set_gemm_pair": [c_int],
    "scmx_set_pdl": [c_int],
    "scmx_set_wait_limit_ns": [ctypes.c_uint64],
    "scmx_set_status_word": [c_vp],
    "scmx_set_gemv_stream": [c_int],
    "scmx_route_sort": [c_vp, c_i64, c_int, c_int, c_int, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp],
    "scmx_router_topk": [c_vp, c_i64, c_int, c_int, c_vp, c_vp, c_vp, c_vp],
    "scmx_gather_rows": [c_vp, c_vp, c_vp, c_i64, c_i64, c_i64, c_vp, c_vp, c_vp],
    "scmx_moe_mm_i8": [c_vp, c_i64, c_vp, c_vp, c_vp, c_vp, c_int, c_i64, c_i64, c_int, c_vp, c_vp, c_int, c_vp, c_vp],
    "scmx_moe_mm": [c_vp, c_i64, c_vp, c_vp, c_vp, c_vp, c_vp, c_int, c_i64, c_i64, _FMT_P, c_int, c_vp, c_vp, c_int,
                    c_int, c_vp, c_i64, c_vp, c_vp],
    "scmx_moe_mm_static": [c_vp, c_i64, c_vp, c_vp, c_vp, c_vp, c_vp, c_int, c_i64, c_i64, _FMT_P, c_int, c_vp, c_vp, c_int,
                           c_vp, c_vp],
    "scmx_ep_dispatch": [c_vp, c_vp, c_vp, c_vp, c_vp, c_i64, c_i64, c_int, c_int, c_int, c_i64, c_vp, c_vp, c_vp, c_vp],
    "scmx_peer_put": [c_vp, c_i64, c_i64, c_vp, c_int, c_vp],
    "scmx_peer_barrier": [c_vp, c_int, c_int, c_vp, c_vp, c_vp],
    "scmx_ep_plan": [c_vp, c_int, c_int, c_i64, c_int, c_i64, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp],
    "scmx_ep_return": [c_vp, c_vp, c_vp, c_vp, c_i64, c_i64, c_int, c_vp, c_vp],
    "scmx_gather_rows_dyn": [c_vp, c_vp, c_vp, c_vp, c_i64, c_int, c_i64, c_vp, c_vp, c_vp],
    "scmx_act_quant_dyn": [c_vp, c_vp, c_i64, c_int, c_i64, c_vp, c_vp, c_vp],
    "scmx_enable_peer_access": [c_int],
    "scmx_moe_mm_i8_ret": [c_vp, c_i64, c_vp, c_vp, c_vp, c_vp, c_int, c_i64, c_i64, c_vp, c_vp, c_vp, c_int, c_vp, c_int, c_vp,
                           c_vp],
    "scmx_moe_combine_pull": [c_vp, c_int, c_int, c_int, c_i64, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_float, c_i64, c_i64, c_i64,
                              c_int, c_int, c_vp, c_vp, c_vp, c_vp],
    "scmx_moe_combine": [c_vp, c_vp, c_vp, c_vp, c_vp, c_float, c_i64, c_i64, c_i64, c_int, c_int, c_vp, c_vp, c_vp,
                         c_vp],
    "scmx_decode_step_dense": [c_vp, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_float, c_vp, c_vp, c_i64, c_i64, c_vp,
                               c_vp, c_vp, c_vp, c_vp, c_vp, c_int, c_vp, c_vp, c_vp, c_vp],
    "scmx_set_decode_trace": [c_vp, c_int],
    "scmx_gemv_pro": [c_vp, c_int, c_vp, c_float, c_vp, c_vp, c_vp, c_i64, c_i64, _FMT_P, c_int, c_vp, c_vp, c_int, c_int, c_int,
                      c_vp, c_int, c_vp],
    "scmx_gemv_multi_plan": [c_vp, c_int, _FMT_P],
    "scmx_gemv_multi": [c_vp, c_vp, c_int, _FMT_P, c_vp, c_int, c_vp],
    "scmx_gemv": [c_vp, c_vp, c_vp, c_vp, c_vp, c_i64, c_i64, _FMT_P, c_int, c_vp, c_vp, c_int, c_int, c_int, c_vp,
                  c_int, c_vp],
}
_RESTYPE = {"scmx_last_error_string": ctypes.c_char_p}

_lib = None


def lib():
    """The loaded library; raises ImportError with build instructions when it has not been compiled."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(f"{LIB_PATH} is missing: build it with `python {os.path.join(_HERE, 'build.py')}` "
                              "(nvcc, sm_100a). This package has no fallback path.")
        h = ctypes.CDLL(LIB_PATH)
        for name, args in SIGNATURES.items():
            fn = getattr(h, name)
            fn.argtypes = args
            fn.restype = _RESTYPE.get(name, c_int)
        _lib = h
    return _lib


def check(rc):
    if rc != 0:
        raise ScmxError(f"libscmx error {rc}: {lib().scmx_last_error_string().decode()}")


def call(name, *args):
    check(getattr(lib(), name)(*args))


def ptr(t):
    """Device pointer of a tensor (None -> NULL)."""
    return None if t is None else c_vp(t.data_ptr())


def stream():
    return c_vp(torch.cuda.current_stream().cuda_stream)


def require_cuda(*tensors):
    for t in tensors:
        if t is not None and not (isinstance(t, torch.Tensor) and t.is_cuda and t.is_contiguous()):
            raise TypeError("expected contiguous CUDA tensors; this package has no CPU path")


_status = {}


def status_buffer():
    """Per-device int32[4] word the tensor-core kernels write when one of their bounded waits runs out."""
    dev = torch.cuda.current_device()
    if dev not in _status:
        _status[dev] = torch.zeros(4, dtype=torch.int32, device=f"cuda:{dev}")
        with torch.cuda.device(dev):      # kernels whose entry point takes no status argument report here too
            call("scmx_set_status_word", c_vp(_status[dev].data_ptr()))
    return _status[dev]


def check_status():
    """Synchronises and raises if any kernel since the last check gave up on a wait. Call outside timed regions."""
    st = status_buffer()
    v = st.cpu().tolist()
    if v[0] != 0:
        st.zero_()
        raise ScmxError(f"device-side wait ran out: {describe_status(v[0])} (CTA or rank {v[1]}, thread {v[2]})")


_GEMM_ROLES = {6: "GEMM unpack warp waiting for a packed weight tile", 1: "GEMM producer waiting for a free stage", 2: "GEMM MMA warp waiting for a free accumulator",
               3: "GEMM MMA warp waiting for operands", 4: "GEMM epilogue waiting for an accumulator",
               5: "GEMM CTA pair waiting for its peer", 11: "streaming GEMV producer waiting for a free stage",
               12: "streaming GEMV consumer waiting for a tile", 20: "peer barrier waiting for another rank's flag"}


def describe_status(code):
    """Text for a status-word code: 1..5 GEMM roles, 11 / 12 streaming GEMV, 20 peer barrier, 100 + k = grid barrier k of
    the one-kernel decode step."""
    if code >= 100:
        return f"decode step: grid barrier {code - 100} timed out"
    return _GEMM_ROLES.get(code, f"code {code}")
