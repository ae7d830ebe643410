"""ctypes binding of libtlaloc_kernels.so (the C ABI in include/tlaloc_b200.h).

There is no fallback: if the library is missing and cannot be built, importing the ops raises.
"""
from __future__ import annotations

import ctypes
import os
import re

from . import build as _build

F32, BF16, S8, S32, F8E4M3FN = 11, 16, 2, 4, 20
OK, INVALID_ARGUMENT, UNSUPPORTED, INTERNAL = 0, -1, -2, -3
GEMM_EXACT, GEMM_X_F32_EXACT, GEMM_WEIGHTS_CONST, GEMM_I8_MMA, GEMM_X_PLANES = 1, 2, 4, 8, 16

_lib = None

_vp, _i32, _f32, _sz = ctypes.c_void_p, ctypes.c_int32, ctypes.c_float, ctypes.c_size_t

_SIGNATURES = {
    "tlaloc_b200_abi_version": (ctypes.c_int, []),
    "tlaloc_b200_last_error": (ctypes.c_char_p, []),
    "tlaloc_b200_init": (ctypes.c_int, []),
    "tlaloc_b200_launch_count": (ctypes.c_longlong, []),
    "tlaloc_b200_device_status": (ctypes.c_int, []),
    "tlaloc_b200_set_order_faithful": (ctypes.c_int, [ctypes.c_int]),
    "tlaloc_b200_paged_attention_splits": (ctypes.c_int, [_i32] * 5),
    "tlaloc_b200_paged_attention_scratch_bytes": (_sz, [_i32] * 4),
    "tlaloc_b200_paged_attention": (ctypes.c_int, [_vp, _i32, _vp, _vp, _i32, _vp, _vp, _vp, _i32, _vp, _i32, _vp, _vp,
                                                   _i32, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _f32, _i32,
                                                   _vp]),
    "tlaloc_b200_paged_attention_static_scratch_bytes": (_sz, []),
    "tlaloc_b200_paged_attention_static": (ctypes.c_int, [_vp, _i32, _vp, _vp, _i32, _vp, _vp, _vp, _i32, _vp, _i32, _vp,
                                                          _i32, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _f32, _i32,
                                                          _vp]),
    "tlaloc_b200_kv_cache_write": (ctypes.c_int, [_vp, _i32, _vp, _i32, _vp, _i32, _i32, _i32, _vp]),
    "tlaloc_b200_int8_gemm_scratch_bytes": (_sz, [_i32] * 3),
    "tlaloc_b200_int8_gemm": (ctypes.c_int, [_vp, _i32, _vp, _vp, _vp, _vp, _i32, _vp, _sz, _i32, _i32, _i32, _i32, _vp]),
    "tlaloc_b200_int8_gemm_swiglu": (ctypes.c_int, [_vp, _i32, _vp, _vp, _vp, _i32, _vp, _sz, _i32, _i32, _i32, _i32, _vp]),
    "tlaloc_b200_dense_gemm_exact": (ctypes.c_int, [_vp, _i32, _vp, _i32, _vp, _i32, _i32, _i32, _i32, _vp]),
    "tlaloc_b200_embedding": (ctypes.c_int, [_vp, _i32, _vp, _vp, _i32, _i32, _i32, _vp]),
    "tlaloc_b200_rmsnorm": (ctypes.c_int, [_vp, _vp, _vp, _i32, _i32, _i32, _f32, _vp]),
    "tlaloc_b200_rmsnorm_planes": (ctypes.c_int, [_vp, _vp, _vp, _vp, _sz, _i32, _i32, _f32, _vp]),
    "tlaloc_b200_rope_kv_write": (ctypes.c_int, [_vp] * 8 + [_i32, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _vp]),
    "tlaloc_b200_swiglu": (ctypes.c_int, [_vp, _vp, _i32, _vp, _i32, _i32, _i32, _vp]),
    "tlaloc_b200_argmax": (ctypes.c_int, [_vp, _vp, _i32, _i32, _vp]),
    "tlaloc_b200_peer_alloc": (ctypes.c_int, [_sz, ctypes.POINTER(_vp), ctypes.c_char_p]),
    "tlaloc_b200_peer_open": (ctypes.c_int, [ctypes.c_char_p, ctypes.POINTER(_vp)]),
    "tlaloc_b200_peer_close": (ctypes.c_int, [_vp]),
    "tlaloc_b200_peer_free": (ctypes.c_int, [_vp]),
    "tlaloc_b200_peer_allreduce_f32": (ctypes.c_int, [ctypes.POINTER(_vp), _sz, _sz, _vp, _i32, _i32, _sz, _vp]),
    "tlaloc_b200_peer_allreduce_rmsnorm_f32": (ctypes.c_int, [ctypes.POINTER(_vp), _sz, _sz, _sz, _vp, _vp, _f32, _i32, _i32,
                                                              _i32, _i32, _vp]),
    "tlaloc_b200_peer_reduce_rmsnorm_rows_f32": (ctypes.c_int, [ctypes.POINTER(_vp), _sz, _sz, _sz, _vp, _vp, _vp, _f32, _i32, _i32,
                                                               _i32, _i32, _i32, _vp]),
    "tlaloc_b200_peer_sum_rows_f32": (ctypes.c_int, [ctypes.POINTER(_vp), _sz, _sz, _vp, _vp, _vp, _vp, _vp, _f32, _i32, _i32, _i32, _i32, _vp, _sz, _vp]),
    "TlalocRegisterKernels": (ctypes.c_char_p, [_vp]),
    "tlaloc_b200_ffi_handler": (_vp, [ctypes.c_char_p]),
}


def library_path() -> str:
    return _build.LIB


def declared_symbols() -> list[str]:
    """Every function include/tlaloc_b200.h declares."""
    with open(os.path.join(_build.INCLUDE, "tlaloc_b200.h")) as f:
        text = re.sub(r"/\*.*?\*/", "", f.read(), flags=re.S)
    return sorted(set(re.findall(r"\b(tlaloc_b200_\w+|TlalocRegisterKernels)\s*\(", text)))


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        path = _build.build()
        if not os.path.exists(path):
            raise RuntimeError(f"{path} is missing: the CUDA extension has not been built (python -m tlaloc_b200.build)")
        _lib = ctypes.CDLL(path)
        for name, (res, args) in _SIGNATURES.items():
            fn = getattr(_lib, name)
            fn.restype, fn.argtypes = res, args
    return _lib


class KernelError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(message)
        self.status = status


def check(status: int) -> None:
    if status != OK:
        raise KernelError(status, lib().tlaloc_b200_last_error().decode())
