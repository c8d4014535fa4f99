"""ctypes binding of libalignedkv_b200.so (the C ABI declared in include/alignedkv_b200.h).

There is no CPU or PyTorch fallback: if the library is missing or a call fails, an exception is raised.
"""
from __future__ import annotations

import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libalignedkv_b200.so")

# every symbol include/alignedkv_b200.h declares, with its ctypes signature
_P, _I, _F = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
SIGNATURES = {
    "akv_abi_version": (_I, []),
    "akv_last_error": (ctypes.c_char_p, []),
    "akv_set_tuning": (_I, [ctypes.c_char_p, _I]),
    "akv_device_error_flag": (_I, []),
    "akv_device_error_clear": (_I, []),
    "akv_launch_count": (ctypes.c_longlong, []),
    "akv_k_cache_save": (_I, [_P] * 4 + [_I] * 8 + [_P]),
    "akv_k_cache_compute": (_I, [_P] * 7 + [_I] * 7 + [_F, _I, _P]),
    "akv_v_cache_save": (_I, [_P] * 4 + [_I] * 7 + [_P]),
    "akv_v_cache_test_compute": (_I, [_P] * 6 + [_I] * 5 + [_P]),
    "akv_v_cache_compute": (_I, [_P] * 6 + [_I] * 7 + [_P]),
    "akv_decode_step": (_I, [_P] * 15 + [ctypes.c_longlong] + [_I] * 7 + [_P]),
    "akv_decode_step_noalloc": (_I, [_P] * 14 + [_I] * 7 + [_P]),
    "akv_decode_scratch_bytes": (ctypes.c_longlong, [_I] * 4),
    "akv_k_cache_compute_gqa": (_I, [_P] * 7 + [_I] * 8 + [_F, _I, _P]),
    "akv_v_cache_compute_gqa": (_I, [_P] * 7 + [ctypes.c_longlong] + [_I] * 8 + [_P]),
    "akv_v_cache_compute_scratch_bytes": (ctypes.c_longlong, [_I] * 4),
    "akv_decode_step_ex": (_I, [_P] * 16 + [ctypes.c_longlong] + [_I] * 8 + [_P]),
    "akv_decode_scratch_bytes_ex": (ctypes.c_longlong, [_I] * 6),
    "akv_decode_step_masked": (_I, [_P] * 16 + [ctypes.c_longlong, _P, ctypes.c_longlong] + [_I] * 8 + [_P]),
    "akv_shard_step": (_I, [_P] * 16 + [ctypes.c_longlong] + [_I] * 13 + [_P]),
    "akv_lse_merge": (_I, [_P] * 2 + [_I] * 3 + [_P]),
    "akv_exchange_bytes": (ctypes.c_longlong, [_I] * 3),
    "akv_peer_alloc": (_I, [ctypes.c_longlong, ctypes.POINTER(ctypes.c_void_p), _P]),
    "akv_peer_open": (_I, [_P, ctypes.POINTER(ctypes.c_void_p)]),
    "akv_peer_close": (_I, [_P]),
    "akv_peer_free": (_I, [_P]),
    "akv_exchange_merge": (_I, [ctypes.POINTER(ctypes.c_void_p), _I, _I, _P, _P, _I, _I, ctypes.c_uint, _I, _P]),
    "akv_decode_step_exchange": (_I, [_P] * 16 + [ctypes.c_longlong] + [_I] * 8 + [ctypes.POINTER(ctypes.c_void_p), _I, _I,
                                                                               ctypes.c_uint, _I, _P]),
    "akv_rollback": (_I, [_P] * 6 + [_I] * 6 + [_P]),
    "akv_prefill": (_I, [_P] * 13 + [ctypes.c_longlong] + [_I] * 5 + [_P]),
    "akv_prefill_scratch_bytes": (ctypes.c_longlong, [_I] * 4),
    "akv_timing_reset": (_I, []),
    "akv_timing_read": (_I, [ctypes.POINTER(ctypes.c_double), ctypes.POINTER(ctypes.c_double)]),
}

_lib = None


class AlignedKVError(RuntimeError):
    """A C-ABI call returned a negative AKV_ERR_* code."""

    def __init__(self, fn: str, code: int, text: str):
        super().__init__(f"{fn} failed with code {code}: {text}")
        self.code = code


def load() -> ctypes.CDLL:
    """Load the shared library (once).  Raises if it has not been built: the product has no fallback path."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m alignedkv_b200.build` "
                "(alignedkv_b200 has no CPU or PyTorch fallback)")
        lib = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def check(fn: str, code: int) -> None:
    if code != 0:
        raise AlignedKVError(fn, code, load().akv_last_error().decode("utf-8", "replace"))
