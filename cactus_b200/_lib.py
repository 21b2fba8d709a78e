"""ctypes binding of libcactus_b200.so (include/cactus_b200.h).  No fallback: a missing library is an error."""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "lib", "libcactus_b200.so")

_i64, _i32, _f32, _vp, _sz = C.c_int64, C.c_int, C.c_float, C.c_void_p, C.c_size_t

# name -> (restype, argtypes); the same list the header declares, checked by tests/test_abi.py
SIGNATURES = {
    "b200_abi_version": (_i32, []),
    "b200_last_error": (C.c_char_p, []),
    "b200_device_count": (_i32, []),
    "b200_device_info": (_i32, [_i32, C.c_char_p, _sz, C.POINTER(_sz), C.POINTER(_sz), C.POINTER(_i32)]),
    "b200_launch_count": (C.c_uint64, []),
    "b200_kernel_status": (C.c_int, []),
    "b200_kernel_set_wait_limit": (None, [C.c_uint]),
    "b200_weight_bytes": (_sz, [_i32, _i64, _i64]),
    "b200_weight_upload": (_i32, [_i32, _i64, _i64, _vp, _vp, _i64, _i64, _vp]),
    "b200_weight_download": (_i32, [_i32, _i64, _i64, _vp, _vp, _i64, _i64, _vp]),
    "b200_quantize_q8_0": (_i32, [_vp, _i64, _i64, _i64, _vp, _i32, _vp]),
    "b200_act_bytes": (_sz, [_i64, _i64]),
    "b200_mul_mat_workspace_bytes": (_sz, [_i32, _i64, _i64, _i64]),
    "b200_mul_mat_scratch_bytes": (_sz, [_i32, _i64, _i64, _i64]),
    "b200_mul_mat_q": (_i32, [_i32, _vp, _i64, _i64, _vp, _i64, _i64, _vp, _i64, _vp, _sz, _i32, _vp]),
    "b200_quantize_activations": (_i32, [_vp, _i64, _i64, _i64, _vp, _sz, _i32, _vp]),
    "b200_mul_mat_q_prequant": (_i32, [_i32, _vp, _i64, _i64, _vp, _i64, _vp, _i64, _vp, _sz, _vp]),
    "b200_mul_mat_q_prequant_multi": (_i32, [_i32, _i32, C.POINTER(_vp), C.POINTER(_i64), _i64, _vp, _i64, C.POINTER(_vp), _i64, _vp, _sz, _vp]),
    "b200_mul_mat_q_noalloc": (_i32, [_i32, _vp, _i64, _i64, _vp, _i64, _i64, _vp, _i64, _i32, _vp]),
    "b200_block_dots": (_i32, [_i32, _vp, _i64, _i64, _vp, _i64, _i64, _vp, _vp, _sz, _i32, _vp]),
    "b200_flash_attn_scratch_bytes": (_sz, [_i64, _i64, _i64, _i64, _i64]),
    "b200_flash_attn_ext": (_i32, [_i64, _i64, _i64, _i64, _i64, _vp, _i64, _i64, _vp, _i64, _i64, _vp, _i64, _i64, _vp, _i64,
                                   _f32, _f32, _f32, _vp, _vp, _sz, _vp]),
    "b200_mask_index_bytes": (_sz, [_i64, _i64]),
    "b200_mask_index_build": (_i32, [_vp, _i64, _i64, _i64, _vp, _sz, _vp]),
    "b200_flash_attn_ext_indexed": (_i32, [_i64, _i64, _i64, _i64, _i64, _vp, _i64, _i64, _vp, _i64, _i64, _vp, _i64, _i64, _vp,
                                           _i64, _vp, _f32, _f32, _f32, _vp, _vp, _sz, _vp]),
    "b200_flash_attn_ext_quant": (_i32, [_i64, _i64, _i64, _i64, _i64, _vp, _i64, _i64, _vp, _i64, _i64, _vp, _i64, _i64, _vp,
                                         _i64, _vp, _f32, _f32, _f32, _vp, _vp, _sz, _i32, _vp, _sz, _vp]),
    "b200_flash_attn_ext_parity": (_i32, [_i64, _i64, _i64, _i64, _i64, _vp, _i64, _i64, _vp, _i64, _i64, _vp, _i64, _i64, _vp,
                                          _i64, _vp, _f32, _f32, _f32, _vp, _vp]),
    "b200_rms_norm": (_i32, [_vp, _i64, _vp, _vp, _i64, _i64, _i64, _f32, _vp]),
    "b200_add": (_i32, [_vp, _vp, _vp, _i64, _i64, _i64, _vp]),
    "b200_mul": (_i32, [_vp, _vp, _vp, _i64, _i64, _i64, _vp]),
    "b200_silu": (_i32, [_vp, _vp, _vp, _i64, _vp]),
    "b200_rope_norm": (_i32, [_vp, _i64, _i64, _vp, _i64, _i64, _i64, _i64, _i64, _i32, _vp, _vp, _f32, _f32, _f32, _vp]),
    "b200_rope_norm_f16": (_i32, [_vp, _i64, _i64, _vp, _i64, _i64, _i64, _i64, _i64, _i32, _vp, _vp, _f32, _f32, _f32, _vp]),
    "b200_cpy_f16_f16": (_i32, [_vp, _i64, _vp, _i64, _i64, _i64, _vp]),
    "b200_cpy_f32_f16": (_i32, [_vp, _i64, _vp, _i64, _i64, _i64, _vp]),
    "b200_cpy_f32_f32": (_i32, [_vp, _i64, _vp, _i64, _i64, _i64, _vp]),
    "b200_get_rows_f32": (_i32, [_vp, _i64, _vp, _vp, _i64, _i64, _i64, _vp]),
    "b200_get_rows_q": (_i32, [_i32, _vp, _i64, _i64, _vp, _vp, _i64, _i64, _vp]),
    "b200_kq_mask_build": (_i32, [_vp, _vp, _i64, _vp, _vp, _i64, _vp, _i64, _vp]),
    "b200_scatter_i32": (_i32, [_vp, _vp, _vp, _i64, _vp]),
    "b200_set_rows_f16": (_i32, [_vp, _i64, _vp, _vp, _i64, _i64, _i64, _vp]),
    "b200_argmax_rows": (_i32, [_vp, _i64, _i64, _i64, _vp, _vp]),
    "b200_add_rms_norm_quantize": (_i32, [_vp, _i64, _vp, _i64, _vp, _vp, _i64, _i64, _i64, _f32, _vp, _sz, _i32, _vp]),
    "b200_silu_mul_quantize": (_i32, [_vp, _vp, _i64, _vp, _i64, _i64, _i64, _vp, _sz, _i32, _vp]),
    "b200_rope_store": (_i32, [_vp, _i64, _i64, _vp, _i64, _i64, _vp, _i64, _i64, _i64, _i64, _i64, _i32, _vp, _vp, _f32, _f32, _f32, _vp,
                               _vp, _i64, _vp, _i64, _vp]),
    "b200_rope_store_to": (_i32, [_vp, _vp, _i64, _i64, _vp, _i64, _i64, _vp, _i64, _i64, _i64, _i64, _i64, _i32, _vp, _vp, _f32, _f32, _f32, _vp,
                                  _vp, _i64, _vp, _i64, _vp]),
    "b200_peer_alloc": (_i32, [_sz, C.POINTER(_vp), C.c_char_p]),
    "b200_peer_open": (_i32, [C.c_char_p, C.POINTER(_vp)]),
    "b200_peer_close": (_i32, [_vp]),
    "b200_peer_free": (_i32, [_vp]),
    "b200_allgather_rows": (_i32, [_vp, _i64, _i64, _i64, _i32, _i32, C.POINTER(_vp), _i64, C.POINTER(_vp), _vp]),
    "b200_peer_status": (_i32, [_vp]),
    "b200_peer_set_wait_limit": (_i32, [_vp, C.c_uint]),
    "b200_mul_mat_q_rowsplit": (_i32, [_i32, _vp, _i64, _i64, _vp, _i64, _i32, _i32, C.POINTER(_vp), _i64, _i64, _vp, _sz, C.POINTER(_vp), _vp]),
    "b200_mul_mat_q_rowsplit_stacked": (_i32, [_i32, _vp, _i64, _i64, _vp, _i64, _i32, _i32, C.POINTER(_vp), _i64, _i32, C.POINTER(_i64), C.POINTER(_i64),
                                               _vp, _sz, C.POINTER(_vp), _vp]),
}

_lib = None


class B200Error(RuntimeError):
    pass


def lib() -> C.CDLL:
    """Loads the kernel library.  Raises if it has not been built: there is no other compute path."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise B200Error(f"{LIB_PATH} is missing: build it with `python -m cactus_b200.build` (needs nvcc); "
                            "cactus_b200 has no CPU or framework fallback")
        L = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        if L.b200_abi_version() != 1:
            raise B200Error("libcactus_b200.so has an unexpected ABI version")
        _lib = L
    return _lib


def check(rc: int) -> None:
    if rc != 0:
        raise B200Error(f"cactus_b200 error {rc}: {lib().b200_last_error().decode()}")
