"""numpy/ctypes access to the CPU checkers.  TEST INFRASTRUCTURE ONLY.

Two libraries live beside this file:

* ``liboracle.so``  -- the plain-C restatement (oracle.c); always buildable with gcc.
* ``_ref/libref_ops.so`` -- the reference's own ggml-cpu compiled from its sources plus a small shim
  (ref_ops.cpp); present only where it was built from a checkout of the reference.

Only tests, the smoke check and the CPU-baseline leg of the benchmark import this module.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
Q4_0, Q8_0 = 2, 8
BLOCK_BYTES = {Q4_0: 18, Q8_0: 34}
Q8_AVX2, Q8_SCALAR = 0, 1

_f32p = np.ctypeslib.ndpointer(np.float32, flags="C_CONTIGUOUS")
_u8p = np.ctypeslib.ndpointer(np.uint8, flags="C_CONTIGUOUS")
_u16p = np.ctypeslib.ndpointer(np.uint16, flags="C_CONTIGUOUS")
_i32p = np.ctypeslib.ndpointer(np.int32, flags="C_CONTIGUOUS")


def build_oracle() -> str:
    path = os.path.join(HERE, "liboracle.so")
    src = [os.path.join(HERE, f) for f in ("oracle.c", "oracle.h")]
    if not os.path.exists(path) or any(os.path.getmtime(s) > os.path.getmtime(path) for s in src):
        subprocess.check_call(["make", "-C", HERE, "oracle"], stdout=subprocess.DEVNULL)
    return path


def default_reference_root() -> str:
    """A checkout of the reference: $CACTUS_REFERENCE, else the directory "reference/cactus" beside this repository."""
    return os.environ.get("CACTUS_REFERENCE") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference", "cactus")


def build_ref(reference_root: str | None = None) -> str | None:
    """Compile the reference from its own sources when a checkout is present; otherwise use what is there."""
    reference_root = reference_root or default_reference_root()
    path = os.path.join(HERE, "_ref", "libref_ops.so")
    if os.path.isdir(reference_root):
        subprocess.check_call(["make", "-C", HERE, "-j8", "ref", f"REF={reference_root}"], stdout=subprocess.DEVNULL)
    return path if os.path.exists(path) else None


class Oracle:
    def __init__(self):
        L = C.CDLL(build_oracle())
        self.L = L
        i64, f32, i32 = C.c_int64, C.c_float, C.c_int
        L.orc_fp32_to_fp16.restype = C.c_uint16
        L.orc_fp32_to_fp16.argtypes = [f32]
        L.orc_fp16_to_fp32.restype = f32
        L.orc_fp16_to_fp32.argtypes = [C.c_uint16]
        L.orc_quantize_row_q4_0.argtypes = [_f32p, _u8p, i64]
        L.orc_quantize_row_q8_0.argtypes = [_f32p, _u8p, i64, i32]
        L.orc_dequantize_row_q4_0.argtypes = [_u8p, _f32p, i64]
        L.orc_dequantize_row_q8_0.argtypes = [_u8p, _f32p, i64]
        L.orc_block_dots.argtypes = [i32, i64, C.c_void_p, C.c_void_p, _i32p]
        L.orc_vec_dot.restype = f32
        L.orc_vec_dot.argtypes = [i32, i64, C.c_void_p, C.c_void_p]
        L.orc_mul_mat.argtypes = [i32, i64, i64, i64, _u8p, C.c_void_p, i64, _f32p, C.c_void_p, i32]
        L.orc_flash_attn_ext.argtypes = [i64, i64, i64, i64, i64, _f32p, _u16p, _u16p, _u16p, f32, f32, f32, _f32p, i32]
        L.orc_build_kq_mask.argtypes = [i64, i64, _i32p, _i32p, _i32p, _i32p, _u16p]
        L.orc_rms_norm_mul.argtypes = [i64, i64, _f32p, _f32p, f32, _f32p]
        L.orc_silu_mul.argtypes = [i64, _f32p, _f32p, _f32p]
        L.orc_add.argtypes = [i64, _f32p, _f32p, _f32p]
        L.orc_rope_norm.argtypes = [i64, i64, i64, _f32p, _i32p, f32, _f32p]
        L.orc_cpy_f32_f16.argtypes = [i64, _f32p, _u16p]
        L.orc_rope_norm_f16.argtypes = [i64, i64, i64, _u16p, _i32p, f32, _u16p]
        L.orc_get_rows.argtypes = [i32, i64, i64, _u8p, _i32p, _f32p]

    # ---- quantisers -------------------------------------------------------------------------
    def quantize_weights(self, wtype: int, w: np.ndarray) -> np.ndarray:
        """w f32 [M, K] -> uint8 [M, K/32*block_bytes] (Q8_0 weights use the scalar variant, as the
        reference's lm_ggml_quantize_chunk does)."""
        w = np.ascontiguousarray(w, np.float32)
        M, K = w.shape
        out = np.empty((M, K // 32 * BLOCK_BYTES[wtype]), np.uint8)
        for m in range(M):
            if wtype == Q4_0:
                self.L.orc_quantize_row_q4_0(w[m], out[m], K)
            else:
                self.L.orc_quantize_row_q8_0(w[m], out[m], K, Q8_SCALAR)
        return out

    def quantize_q8_0(self, x: np.ndarray, variant: int = Q8_AVX2) -> np.ndarray:
        x = np.ascontiguousarray(x, np.float32)
        N, K = x.shape
        out = np.empty((N, K // 32 * 34), np.uint8)
        for n in range(N):
            self.L.orc_quantize_row_q8_0(x[n], out[n], K, variant)
        return out

    def dequantize(self, wtype: int, wq: np.ndarray, K: int) -> np.ndarray:
        M = wq.shape[0]
        out = np.empty((M, K), np.float32)
        fn = self.L.orc_dequantize_row_q4_0 if wtype == Q4_0 else self.L.orc_dequantize_row_q8_0
        for m in range(M):
            fn(np.ascontiguousarray(wq[m]), out[m], K)
        return out

    # ---- dots -------------------------------------------------------------------------------
    def block_dots(self, wtype: int, wq: np.ndarray, aq: np.ndarray, K: int) -> np.ndarray:
        """int32 [N, M, K/32]: exact per-block integer dots."""
        M, N = wq.shape[0], aq.shape[0]
        out = np.empty((N, M, K // 32), np.int32)
        for n in range(N):
            for m in range(M):
                self.L.orc_block_dots(wtype, K, wq[m].ctypes.data, aq[n].ctypes.data, out[n, m])
        return out

    def mul_mat(self, wtype: int, wq: np.ndarray, x: np.ndarray, variant: int = Q8_AVX2):
        """returns (dst f32 [N, M], q8 uint8 [N, K/32*34])"""
        x = np.ascontiguousarray(x, np.float32)
        wq = np.ascontiguousarray(wq)
        N, K = x.shape
        M = wq.shape[0]
        dst = np.empty((N, M), np.float32)
        q8 = np.empty((N, K // 32 * 34), np.uint8)
        self.L.orc_mul_mat(wtype, M, K, N, wq, x.ctypes.data, K, dst, q8.ctypes.data, variant)
        return dst, q8

    # ---- attention --------------------------------------------------------------------------
    def flash_attn_ext(self, q, kc, vc, mask, scale, max_bias=0.0, softcap=0.0, n_kv=None, acc_mode=0):
        """q f32 [Nq,H,D]; kc, vc uint16 [cells,Hkv,D]; mask uint16 [pad64(Nq), n_kv] -> f32 [Nq,H,D]"""
        Nq, H, D = q.shape
        Hkv = kc.shape[1]
        n_kv = kc.shape[0] if n_kv is None else n_kv
        dst = np.empty((Nq, H, D), np.float32)
        self.L.orc_flash_attn_ext(D, H, Hkv, Nq, n_kv, np.ascontiguousarray(q, np.float32), np.ascontiguousarray(kc),
                                  np.ascontiguousarray(vc), np.ascontiguousarray(mask), scale, max_bias, softcap, dst, acc_mode)
        return dst

    def build_kq_mask(self, n_kv, cell_pos, cell_seq, tok_pos, tok_seq):
        T = len(tok_pos)
        mask = np.empty(((T + 63) // 64 * 64, n_kv), np.uint16)
        self.L.orc_build_kq_mask(n_kv, T, np.ascontiguousarray(cell_pos, np.int32), np.ascontiguousarray(cell_seq, np.int32),
                                 np.ascontiguousarray(tok_pos, np.int32), np.ascontiguousarray(tok_seq, np.int32), mask)
        return mask

    # ---- row ops ----------------------------------------------------------------------------
    def rms_norm_mul(self, x, w, eps):
        T, d = x.shape
        dst = np.empty_like(x)
        self.L.orc_rms_norm_mul(d, T, np.ascontiguousarray(x), np.ascontiguousarray(w), eps, dst)
        return dst

    def silu_mul(self, a, b):
        dst = np.empty_like(a)
        self.L.orc_silu_mul(a.size, np.ascontiguousarray(a), np.ascontiguousarray(b), dst)
        return dst

    def add(self, a, b):
        dst = np.empty_like(a)
        self.L.orc_add(a.size, np.ascontiguousarray(a), np.ascontiguousarray(b), dst)
        return dst

    def rope_norm(self, x, pos, freq_base):
        T, H, D = x.shape
        dst = np.empty_like(x)
        self.L.orc_rope_norm(D, H, T, np.ascontiguousarray(x), np.ascontiguousarray(pos, np.int32), freq_base, dst)
        return dst

    def rope_norm_f16(self, x, pos, freq_base):
        """x uint16 (f16 bits) [T, H, D], pos int32 [T] -> uint16 [T, H, D]"""
        T, H, D = x.shape
        dst = np.empty_like(x)
        self.L.orc_rope_norm_f16(D, H, T, np.ascontiguousarray(x, np.uint16), np.ascontiguousarray(pos, np.int32), freq_base, dst)
        return dst

    def cpy_f32_f16(self, x):
        dst = np.empty(x.shape, np.uint16)
        self.L.orc_cpy_f32_f16(x.size, np.ascontiguousarray(x), dst)
        return dst

    def get_rows(self, wtype, table, ids, d):
        dst = np.empty((len(ids), d), np.float32)
        self.L.orc_get_rows(wtype, d, len(ids), np.ascontiguousarray(table), np.ascontiguousarray(ids, np.int32), dst)
        return dst


class Reference:
    """The reference's own ggml-cpu (oracle/_ref).  ``Reference.load()`` returns None when it is absent."""

    @staticmethod
    def load(build: bool = True):
        path = build_ref() if build else os.path.join(HERE, "_ref", "libref_ops.so")
        if path is None or not os.path.exists(path):
            return None
        return Reference(path)

    def __init__(self, path):
        L = C.CDLL(path)
        self.L = L
        i64, f32, i32, dbl = C.c_int64, C.c_float, C.c_int, C.c_double
        L.ref_init()
        L.ref_quantize_weights.restype = i64
        L.ref_quantize_weights.argtypes = [i32, _f32p, _u8p, i64, i64]
        L.ref_quantize_row_q8_0.argtypes = [_f32p, _u8p, i64]
        L.ref_quantize_row_q8_0_scalar.argtypes = [_f32p, _u8p, i64]
        L.ref_dequantize_row.argtypes = [i32, _u8p, _f32p, i64]
        L.ref_vec_dot.restype = f32
        L.ref_vec_dot.argtypes = [i32, i64, C.c_void_p, C.c_void_p]
        L.ref_mul_mat.restype = dbl
        L.ref_mul_mat.argtypes = [i32, i64, i64, i64, _u8p, C.c_void_p, i64, _f32p, i32, i32, i32]
        L.ref_flash_attn_ext.restype = dbl
        L.ref_flash_attn_ext.argtypes = [i64, i64, i64, i64, i64, _f32p, _u16p, _u16p, _u16p, f32, f32, f32, _f32p, i32, i32, i32]
        L.ref_row_op.argtypes = [i32, i64, i64, i64, C.c_void_p, C.c_void_p, f32, C.c_void_p, i32]

    def quantize_weights(self, wtype, w):
        w = np.ascontiguousarray(w, np.float32)
        M, K = w.shape
        out = np.empty((M, K // 32 * BLOCK_BYTES[wtype]), np.uint8)
        n = self.L.ref_quantize_weights(wtype, w, out, M, K)
        assert n == out.size
        return out

    def quantize_q8_0(self, x, variant=Q8_AVX2):
        x = np.ascontiguousarray(x, np.float32)
        N, K = x.shape
        out = np.empty((N, K // 32 * 34), np.uint8)
        fn = self.L.ref_quantize_row_q8_0 if variant == Q8_AVX2 else self.L.ref_quantize_row_q8_0_scalar
        for n in range(N):
            fn(x[n], out[n], K)
        return out

    def vec_dot(self, wtype, w_row, a_row, K):
        return self.L.ref_vec_dot(wtype, K, w_row.ctypes.data, a_row.ctypes.data)

    def mul_mat(self, wtype, wq, x, n_threads=1, warmup=0, reps=1):
        """returns (dst f32 [N, M], median seconds)"""
        x = np.ascontiguousarray(x, np.float32)
        wq = np.ascontiguousarray(wq)
        N, K = x.shape
        M = wq.shape[0]
        dst = np.empty((N, M), np.float32)
        t = self.L.ref_mul_mat(wtype, M, K, N, wq, x.ctypes.data, K, dst, n_threads, warmup, reps)
        return dst, t

    def flash_attn_ext(self, q, kc, vc, mask, scale, max_bias=0.0, softcap=0.0, n_kv=None, n_threads=1, warmup=0, reps=1):
        Nq, H, D = q.shape
        Hkv = kc.shape[1]
        n_kv = kc.shape[0] if n_kv is None else n_kv
        dst = np.empty((Nq, H, D), np.float32)
        t = self.L.ref_flash_attn_ext(D, H, Hkv, Nq, n_kv, np.ascontiguousarray(q, np.float32), np.ascontiguousarray(kc),
                                      np.ascontiguousarray(vc), np.ascontiguousarray(mask), scale, max_bias, softcap, dst,
                                      n_threads, warmup, reps)
        return dst, t

    def row_op(self, op, a, b, p0=0.0, out_dtype=np.float32):
        a = np.ascontiguousarray(a, np.uint16 if op == 5 else np.float32)   # op 5 takes f16 bits
        if a.ndim == 3:
            T, h, d = a.shape
        else:
            (T, d), h = a.shape, 1
        dst = np.empty(a.shape, out_dtype)
        b = np.ascontiguousarray(b) if b is not None else None
        rc = self.L.ref_row_op(op, d, h, T, a.ctypes.data, b.ctypes.data if b is not None else None, p0, dst.ctypes.data, 1)
        assert rc == 0
        return dst
