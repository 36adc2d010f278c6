"""SC-MXFP4 W4A8 hot path for NVIDIA B200 (sm_100a): quantizer/packer, per-token INT8 activation quantizer, tcgen05
dense and grouped-MoE GEMMs, decode GEMV.  Python modules mirror the reference's e2e/sc_format.py, sc_kernels.py,
sc_moe.py, sc_decode.py and w4a8_mlx.py; all arithmetic runs in libscmx.so (include/scmx.h).  No CPU fallback."""
import sys as _sys

from . import _lib, sc_format, sc_kernels, sc_moe, sc_decode, w4a8, fused_dense, fused_moe, parallel  # noqa: F401
from . import host_model, packed_io, fused_qwen3, fused_olmoe, decode  # noqa: F401

_sys.modules.setdefault("scmx_b200", _sys.modules[__name__])
