"""alignedkv_b200: B200-native (sm_100a) implementation of AlignedKV's decode hot path.

Layout
  csrc/        hand-written CUDA kernels and the extern "C" surface (declared in include/alignedkv_b200.h)
  _lib.py      ctypes binding of libalignedkv_b200.so
  extension/   host-side mirror of the reference's `extension` package: `cuda_module` with the five operators,
               `K_Cache_Class`, `V_Cache_Class` (same names, arguments and error behaviour)

`install_as_extension()` registers the mirror under the reference's import names so that the reference's
model/KVCache_AlignedKV.py imports it unchanged.
"""
from __future__ import annotations

import sys

__all__ = ["install_as_extension"]


def install_as_extension() -> None:
    """Make `import extension.k_cache_file` (the reference's import path, model/KVCache_AlignedKV.py:10-11)
    resolve to this package's mirror modules."""
    from . import extension as ext
    from .extension import KV_cache_cpp_extention, k_cache_file, v_cache_file

    sys.modules["extension"] = ext
    sys.modules["extension.KV_cache_cpp_extention"] = KV_cache_cpp_extention
    sys.modules["extension.k_cache_file"] = k_cache_file
    sys.modules["extension.v_cache_file"] = v_cache_file
