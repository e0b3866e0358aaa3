"""ctypes binding of locomp_b200/_lcq.so (the C ABI in include/locomp_b200.h).

There is no fallback: if the shared library is missing, importing an operator raises.
"""
from __future__ import annotations

import ctypes
import os

from .build import LIB_PATH

OK = 0
ERR_BAD_ARG, ERR_UNSUPPORTED, ERR_CUDA, ERR_WORKSPACE, ERR_TIMEOUT = -1, -2, -3, -4, -5
F32, F16, BF16 = 0, 1, 2
ALGO_AUTO, ALGO_SIMT, ALGO_GEMV_TC, ALGO_GEMM_TC, ALGO_GEMV_W8 = 0, 1, 2, 3, 4

# name -> (restype, argtypes); mirrors include/locomp_b200.h one to one
_c = ctypes
SIGNATURES = {
    "lcq_version": (_c.c_int, []),
    "lcq_status_string": (_c.c_char_p, [_c.c_int]),
    "lcq_last_error": (_c.c_char_p, []),
    "lcq_device_info": (_c.c_int, [_c.c_int, _c.c_char_p, _c.c_size_t, _c.POINTER(_c.c_int),
                                   _c.POINTER(_c.c_int), _c.POINTER(_c.c_int), _c.POINTER(_c.c_int)]),
    "lcq_dequant_int4": (_c.c_int, [_c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_int64, _c.c_int64, _c.c_int,
                                    _c.c_int, _c.c_int, _c.c_void_p]),
    "lcq_dequant_int8": (_c.c_int, [_c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_int64, _c.c_int64, _c.c_int,
                                    _c.c_int, _c.c_int, _c.c_void_p]),
    "lcq_matmul_int4": (_c.c_int, [_c.c_void_p] * 4 + [_c.c_int] * 8 + [_c.c_void_p, _c.c_size_t, _c.c_void_p]),
    "lcq_matmul_int8": (_c.c_int, [_c.c_void_p] * 4 + [_c.c_int] * 8 + [_c.c_void_p, _c.c_size_t, _c.c_void_p]),
    "lcq_matmul_workspace_bytes": (_c.c_size_t, [_c.c_int] * 9),
    "lcq_matmul_select_algo": (_c.c_int, [_c.c_int] * 8),
    "lcq_matmul_int4_noalloc": (_c.c_int, [_c.c_void_p] * 4 + [_c.c_int] * 7 + [_c.c_void_p]),
    "lcq_noalloc_scratch_bytes": (_c.c_size_t, []),
    "lcq_rms_norm": (_c.c_int, [_c.c_void_p] * 3 + [_c.c_int64, _c.c_int, _c.c_float, _c.c_int, _c.c_void_p]),
    "lcq_residual_rms_norm": (_c.c_int, [_c.c_void_p] * 4 + [_c.c_int64, _c.c_int, _c.c_float, _c.c_int, _c.c_void_p]),
    "lcq_silu_mul": (_c.c_int, [_c.c_void_p] * 3 + [_c.c_int64, _c.c_int, _c.c_void_p]),
    "lcq_add_inplace": (_c.c_int, [_c.c_void_p] * 2 + [_c.c_int64, _c.c_int, _c.c_void_p]),
    "lcq_embed_lookup": (_c.c_int, [_c.c_void_p] * 3 + [_c.c_int64, _c.c_int, _c.c_int, _c.c_int, _c.c_void_p]),
    "lcq_argmax": (_c.c_int, [_c.c_void_p] * 2 + [_c.c_int64, _c.c_int, _c.c_int, _c.c_void_p]),
    "lcq_quantize_int4": (_c.c_int, [_c.c_void_p] * 3 + [_c.c_int64, _c.c_int64, _c.c_int, _c.c_int, _c.c_int, _c.c_void_p]),
    "lcq_quantize_int8": (_c.c_int, [_c.c_void_p] * 3 + [_c.c_int64, _c.c_int64, _c.c_int, _c.c_int, _c.c_int, _c.c_void_p]),
    "lcq_peer_alloc": (_c.c_int, [_c.c_size_t, _c.POINTER(_c.c_void_p), _c.c_char_p]),
    "lcq_peer_open": (_c.c_int, [_c.c_char_p, _c.POINTER(_c.c_void_p)]),
    "lcq_peer_close": (_c.c_int, [_c.c_void_p]),
    "lcq_peer_free": (_c.c_int, [_c.c_void_p]),
    "lcq_allgather_push": (_c.c_int, [_c.c_void_p, _c.c_size_t, _c.POINTER(_c.c_void_p), _c.c_int, _c.c_int,
                                      _c.c_void_p, _c.c_void_p]),
    "lcq_peer_region_bytes": (_c.c_size_t, [_c.c_size_t, _c.c_int]),
    "lcq_shard_ctx_create": (_c.c_int, [_c.c_int, _c.c_int, _c.c_size_t, _c.POINTER(_c.c_void_p), _c.c_char_p]),
    "lcq_shard_ctx_connect": (_c.c_int, [_c.c_void_p, _c.c_char_p]),
    "lcq_sharded_matmul_int4": (_c.c_int, [_c.c_void_p] * 4 + [_c.POINTER(_c.c_void_p)] + [_c.c_int] * 8 + [_c.c_void_p]),
    "lcq_shard_ctx_destroy": (_c.c_int, [_c.c_void_p]),
    "lcq_check_device_status": (_c.c_int, [_c.c_void_p]),
    "lcq_set_wait_limit_ns": (_c.c_int, [_c.c_ulonglong]),
    "lcq_gemv_tc_plan_check": (_c.c_int, [_c.c_int] * 4 + [_c.POINTER(_c.c_int)]),
    "lcq_gemv_tc_plan_cluster": (_c.c_int, [_c.c_int] * 4),
}


class LcqError(RuntimeError):
    """A C entry point returned a negative status; carries the status and the library's message."""

    def __init__(self, status: int, message: str):
        super().__init__(f"locomp_b200 status {status}: {message}")
        self.status = status


_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: the CUDA library has not been built "
                "(run `python -m locomp_b200.build`); there is no CPU fallback")
        handle = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)   # AttributeError if the symbol is not exported
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def check(status: int) -> None:
    if status < 0:
        msg = lib().lcq_last_error().decode() or lib().lcq_status_string(status).decode()
        if status == ERR_BAD_ARG:
            raise ValueError(f"locomp_b200: {msg}")
        raise LcqError(status, msg)
