"""CPU: host-side logic of the package (layout helpers, Format checks), the C-ABI library's exports, and the
argument validation every entry point performs before touching the GPU."""
import ctypes
import os
import re

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol(scmx):
    hdr = open(os.path.join(ROOT, "include", "scmx.h")).read()
    declared = set(re.findall(r"\b(scmx_[a-z0-9_]+)\s*\(", hdr))
    assert len(declared) >= 18
    h = ctypes.CDLL(scmx._lib.LIB_PATH)
    for name in declared:
        assert hasattr(h, name), f"{name} declared in include/scmx.h but not exported"
    assert declared == set(scmx._lib.SIGNATURES), "python binding and header disagree"
    assert scmx._lib.lib().scmx_abi_version() == 1


def test_pack_rows_decode_against_reference_vectors(scmx, golden):
    F = scmx.sc_format
    fmt = F.Format(block=16, mult=(1, 2, 3, 4, 5, 6, 8, 10), bc_bits=4)
    cc, bb, _ = F.pack_rows(golden["generic_code4"], golden["generic_bcode"], np.ones(8), fmt)
    assert np.array_equal(cc, golden["generic_codes"]) and np.array_equal(bb, golden["generic_bcodes"])
    assert np.array_equal(F.decode_numpy(cc, bb, 8, 256, fmt), golden["generic_q"])
    for tag in "abc":
        qw = golden[f"quantize_{tag}_qw"]
        assert np.array_equal(F.decode_numpy(golden[f"quantize_{tag}_codes"], golden[f"quantize_{tag}_bcodes"], *qw.shape), qw)


def test_from_shift_layout_roundtrip(scmx, golden):
    F = scmx.sc_format
    bc = golden["quantize_a_bcodes"]
    shifts = ((bc[..., None] >> (2 * np.arange(4, dtype=np.uint8))) & 3).reshape(bc.shape[0], -1)
    c, b, s = F.from_shift_layout(golden["quantize_a_codes"], shifts, golden["quantize_a_wscale"])
    assert np.array_equal(b, bc) and np.array_equal(c, golden["quantize_a_codes"])


def test_format_checks(scmx):
    F = scmx.sc_format
    assert F.DEFAULT.bits_per_weight(4096) == pytest.approx(4 + 2 / 32 + 32 / 4096)
    with pytest.raises(AssertionError):
        F.Format(block=12)
    with pytest.raises(AssertionError):
        F.Format(mult=(1, 2, 4, 8, 16))          # does not fit 2-bit block codes
    with pytest.raises(AssertionError):
        F.Format(mult=(1, 2, 4, 11))             # 12 * 11 > 127
    f = F.Format(block=16, mult=(1, 2, 3, 4, 5, 6, 8, 10), bc_bits=4).c_struct()
    assert (f.block, f.bc_bits, f.n_mult, f.mult[7]) == (16, 4, 8, 10)


def test_interleave_and_padding(scmx, golden):
    S = scmx.sc_kernels
    assert np.array_equal(S.interleave_gate_up(768), golden["perm_768"])
    assert [S.pad_rows(m) for m in (1, 128, 129, 200)] == [128, 128, 256, 256]


def test_entry_points_validate_before_launch(scmx):
    """Bad shapes and formats are rejected on the host with an error string; nothing reaches the GPU."""
    L = scmx._lib
    lib = L.lib()
    fmt = scmx.sc_format.DEFAULT.c_struct()
    bad = scmx.sc_format.DEFAULT.c_struct()
    bad.mult[3] = 11
    assert lib.scmx_act_quant(None, 4, 7, 4, None, None, None) == -1
    assert b"K % 8" in lib.scmx_last_error_string()
    assert lib.scmx_unpack_i8(None, None, 4, 256, bad, None, None) == -2
    assert b"INT8" in lib.scmx_last_error_string()
    assert lib.scmx_quantize_sc_mxfp4(None, 0, 4, 100, None, None, None, None, None, None) == -1
    assert lib.scmx_mm_i8(None, None, 128, 100, 256, 0, None, None, None, None, None, None) == -1
    assert lib.scmx_mm_i8(None, None, 128, 128, 256, 1, None, None, None, ctypes.c_void_p(16), ctypes.c_void_p(16), None) == -1
    assert lib.scmx_gemv(None, None, None, None, None, 6, 256, fmt, 1, None, None, 0, -1, 0, None, 0, None) == -1
    assert lib.scmx_route_sort(None, 4, 2, 2000, 128, None, None, None, None, None, None) == -5
    assert lib.scmx_moe_mm_i8(None, 10, None, None, ctypes.c_void_p(16), ctypes.c_void_p(16), 4, 128, 256, 0, None,
                              ctypes.c_void_p(16), 64, ctypes.c_void_p(16), None) == -1
    assert b"tm=64" in lib.scmx_last_error_string()
    assert lib.scmx_set_gemm_tile(64) == -1 and lib.scmx_set_gemm_tile(0) == 0
    with pytest.raises(L.ScmxError):
        L.call("scmx_act_quant", None, 4, 7, 4, None, None, None)


def test_no_cpu_fallback(scmx):
    import torch
    with pytest.raises(TypeError):
        scmx.sc_kernels.act_quant(torch.zeros(4, 64, dtype=torch.bfloat16))


def test_gemv_list_plan_geometry(scmx):
    """scmx_gemv_multi_plan is host code: tile shapes must respect the stage size (64 KB of codes, 2 KB of block codes), use at
    most 16 consumer warps, and number the tiles of the jobs consecutively.  Pointers only need to be non-NULL and aligned."""
    import ctypes
    L = scmx._lib
    shapes = [(4096, 2048), (2048, 2048), (12288, 2048), (2048, 6144), (100, 1024), (64, 8192), (1024, 3072), (4, 512)]
    jobs = (L.ScmxGemvJob * len(shapes))()
    for rec, (n, k) in zip(jobs, shapes):
        rec.codes = rec.bcodes = rec.wscale = rec.xq = rec.xscale = rec.out = 0x1000
        rec.N, rec.K, rec.epi = n, k, 1
    fmt = scmx.sc_format.DEFAULT.c_struct()
    assert L.lib().scmx_gemv_multi_plan(ctypes.byref(jobs), len(shapes), fmt) == 0, L.lib().scmx_last_error_string()
    tile0 = 0
    for rec, (n, k) in zip(jobs, shapes):
        tr, rg, sk, t0, nt, bcrow, kw = (rec.plan[i] for i in range(7))
        assert tr == 4 * rg and 1 <= rg * sk <= 16 and tr * k // 2 <= 65536 and tr * bcrow <= 2048
        assert kw * sk == k and kw % 32 == 0 and bcrow == k // 128
        assert t0 == tile0 and nt == -(-n // tr)
        tile0 += nt
    assert all(rec.plan[8] == tile0 for rec in jobs)
    assert jobs[0].plan[0] == 64 and jobs[3].plan[1] * jobs[3].plan[2] == 15      # K = 2048: 64-row tiles; K = 6144: 5 x 3 warps
    jobs[1].K = 128                                                                # one block-code byte per row: not a multiple of 4
    assert L.lib().scmx_gemv_multi_plan(ctypes.byref(jobs), len(shapes), fmt) == -5
    jobs[1].K = 100                                                                # not a multiple of 128
    assert L.lib().scmx_gemv_multi_plan(ctypes.byref(jobs), len(shapes), fmt) == -1
    jobs[1].K = 16384                                                              # beyond the activation slot of a stage
    assert L.lib().scmx_gemv_multi_plan(ctypes.byref(jobs), len(shapes), fmt) == -1


def test_packed_weight_gemm_format_rule(scmx):
    """scmx_w4_supported: the block codes of 128 weights must form one field of 8, 16 or 32 bits, K a multiple of 128."""
    F, L = scmx.sc_format, scmx._lib
    ok = lambda fmt, k: L.lib().scmx_w4_supported(fmt.c_struct(), k)   # noqa: E731
    assert ok(F.Format(), 2048) and ok(F.Format(block=16), 768) and ok(F.Format(block=16, mult=(1, 2, 3, 4, 5, 6, 8, 10), bc_bits=4), 2048)
    assert not ok(F.Format(), 2048 + 64)
    assert not ok(F.Format(block=64), 2048)            # 4 bits per 128 weights
    assert ok(F.Format(block=8), 2048)                 # 16 blocks x 2 bits = 32 bits
    assert not ok(F.Format(block=8, mult=(1, 2, 3, 4, 5, 6, 8, 10), bc_bits=4), 2048)      # 64 bits


def test_status_word_codes_have_texts(scmx):
    """Every code a kernel can leave in the status word has a description that names the waiting party (what check_status()
    raises with); unknown codes fall back to the number."""
    L = scmx._lib
    for code, word in ((1, "producer"), (2, "MMA"), (3, "MMA"), (4, "epilogue"), (6, "unpack"), (11, "GEMV"), (12, "GEMV"),
                       (20, "peer barrier")):
        assert word in L.describe_status(code), code
    assert "grid barrier 3" in L.describe_status(103)
    assert L.describe_status(77) == "code 77"
