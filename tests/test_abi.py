"""The C-ABI library loads and exports exactly the symbols include/cactus_b200.h declares (no GPU needed)."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    hdr = open(os.path.join(ROOT, "include", "cactus_b200.h")).read()
    return sorted(set(re.findall(r"B200_API[^;]*?\b(b200_\w+)\s*\(", hdr)))


def test_library_exports_every_declared_symbol():
    from cactus_b200 import LIB_PATH
    from cactus_b200.build import build
    build()
    assert os.path.exists(LIB_PATH)
    L = ctypes.CDLL(LIB_PATH)
    names = declared_symbols()
    assert len(names) >= 30
    for n in names:
        assert hasattr(L, n), f"{n} declared in the header but not exported"


def test_python_binding_covers_the_header():
    from cactus_b200._lib import SIGNATURES
    assert sorted(SIGNATURES) == declared_symbols()


def test_size_queries_and_argument_checks_without_a_gpu():
    from cactus_b200._lib import lib
    L = lib()
    assert L.b200_abi_version() == 1
    # T16 layout: rows padded to 16, blocks to 4; 18 bytes per Q4_0 block, 34 per Q8_0 block
    assert L.b200_weight_bytes(2, 4096, 4096) == 4096 * 128 * 18
    assert L.b200_weight_bytes(8, 2048, 128256) == 128256 * 64 * 34
    assert L.b200_weight_bytes(2, 64, 33) == 48 * 4 * 18
    assert L.b200_weight_bytes(2, 100, 16) == 0      # K not a multiple of 32
    assert L.b200_weight_bytes(3, 128, 16) == 0      # unsupported type
    assert L.b200_act_bytes(4096, 1) == 128 * 256 + 32 * 256
    assert L.b200_mul_mat_scratch_bytes(2, 4096, 4096, 2) == L.b200_act_bytes(4096, 2)   # the GEMV kernel needs no workspace
    assert L.b200_mul_mat_scratch_bytes(2, 4096, 4096, 8) >= L.b200_act_bytes(4096, 8)   # the tensor-core kernel may split K
    # words, word list, counts, token order, plan
    assert L.b200_mask_index_bytes(64, 65536) == 64 * 1024 * 8 + 64 * 1024 * 4 + 256 + 256 + 256
    # invalid arguments are rejected before any CUDA call
    rc = L.b200_mul_mat_q(5, None, 64, 16, None, 256, 1, None, 64, None, 0, 0, None)
    assert rc == -1 and b"bad mul_mat" in L.b200_last_error()
    rc = L.b200_flash_attn_ext(96, 8, 8, 1, 256, None, 0, 0, None, 0, 0, None, 0, 0, None, 0, 1.0, 0.0, 0.0, None, None, 0, None)
    assert rc == -1 and b"head size" in L.b200_last_error()
    # a stacked row-split product: the parts must add up to the weight's rows and all but the last hold whole 16-row tiles
    import ctypes as C
    rows, cols = (C.c_int64 * 2)(24, 40), (C.c_int64 * 2)(0, 128)
    rc = L.b200_mul_mat_q_rowsplit_stacked(2, None, 64, 64, None, 4, 0, 1, None, 1024, 2, rows, cols, None, 0, None, None)
    assert rc == -1 and b"multiple of 16" in L.b200_last_error()
    rows = (C.c_int64 * 2)(32, 16)
    rc = L.b200_mul_mat_q_rowsplit_stacked(2, None, 64, 64, None, 4, 0, 1, None, 1024, 2, rows, cols, None, 0, None, None)
    assert rc == -1 and b"the parts hold 48 rows" in L.b200_last_error()
    # several weights in one launch: 1 to 3 of them, none null
    rc = L.b200_mul_mat_q_prequant_multi(2, 4, None, None, 64, None, 16, None, 1024, None, 0, None)
    assert rc == -1 and b"1 to 3 weights" in L.b200_last_error()
    wp, mp, dp = (C.c_void_p * 2)(None, None), (C.c_int64 * 2)(128, 128), (C.c_void_p * 2)(None, None)
    rc = L.b200_mul_mat_q_prequant_multi(2, 2, wp, mp, 64, None, 16, dp, 1024, None, 0, None)
    assert rc == -1 and b"weight / destination 0" in L.b200_last_error()
    rc = L.b200_mul_mat_q_rowsplit_stacked(2, None, 64, 64, None, 4, 0, 1, None, 1024, 4, rows, cols, None, 0, None, None)
    assert rc == -1 and b"1 to 3 parts" in L.b200_last_error()


def test_missing_library_fails_loudly(monkeypatch):
    import cactus_b200._lib as m
    monkeypatch.setattr(m, "_lib", None)
    monkeypatch.setattr(m, "LIB_PATH", "/nonexistent/libcactus_b200.so")
    with pytest.raises(m.B200Error, match="no CPU or framework fallback"):
        m.lib()


def test_plugin_exports_the_loader_entry_points():
    """libggml-b200.so (built where the reference's headers are) exports what lm_ggml_backend_load looks up."""
    import subprocess
    so = os.path.join(ROOT, "cactus_b200", "lib", "libggml-b200.so")
    if not os.path.exists(so):
        pytest.skip("plug-in not built (needs a checkout of the reference)")
    syms = subprocess.run(["nm", "-D", "--defined-only", so], capture_output=True, text=True).stdout
    for name in ("lm_ggml_backend_init", "lm_ggml_backend_score", "lm_ggml_backend_b200_reg", "lm_ggml_backend_b200_init"):
        assert f" T {name}" in syms, name
