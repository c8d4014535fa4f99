"""alignedkv_b200: B200-native (sm_100a) implementation of AlignedKV's decode hot path.

Layout
  csrc/        hand-written CUDA kernels and the extern "C" surface (declared in include/alignedkv_b200.h)
  _lib.py      ctypes binding of libalignedkv_b200.so
  extension/   host-side mirror of the reference's `extension` package: `cuda_module` with the five operators,
               `K_Cache_Class`, `V_Cache_Class` (same names, arguments and error behaviour)

`install_as_extension()` registers the mirror under the reference's import names so that the reference's
model/KVCache_AlignedKV.py imports it unchanged; `load_reference_cache(root)` does that import from a checkout of the
reference and returns its `QuantizedCache_AlignedKV` class.
"""
from __future__ import annotations

import importlib.util
import os
import sys

__all__ = ["install_as_extension", "load_reference_cache"]


def install_as_extension() -> None:
    """Make `import extension.k_cache_file` (the reference's import path, model/KVCache_AlignedKV.py:10-11)
    resolve to this package's mirror modules."""
    from . import extension as ext
    from .extension import KV_cache_cpp_extention, k_cache_file, v_cache_file

    sys.modules["extension"] = ext
    sys.modules["extension.KV_cache_cpp_extention"] = KV_cache_cpp_extention
    sys.modules["extension.k_cache_file"] = k_cache_file
    sys.modules["extension.v_cache_file"] = v_cache_file


def load_reference_cache(reference_root: str):
    """Import the reference's own cache orchestration (model/KVCache_AlignedKV.py, unchanged, from a checkout at
    `reference_root`) on top of this package's operators and return its `QuantizedCache_AlignedKV` class.

    Two things are arranged around the import and nothing in the file is touched: its `extension.*` imports
    (model/KVCache_AlignedKV.py:10-11) resolve to the mirror modules, and, because the class was written for
    transformers 4.44 whose `Cache.__init__` takes no arguments while later releases require layer descriptions and
    make `max_batch_size` / `max_cache_len` read-only properties (both clash with model/KVCache_AlignedKV.py:19-22),
    `transformers.cache_utils.Cache` is a plain base class for the duration of the import."""
    path = os.path.join(reference_root, "model", "KVCache_AlignedKV.py")
    if not os.path.exists(path):
        raise FileNotFoundError(path)
    install_as_extension()
    import transformers.cache_utils as cache_utils

    class _PlainCache:
        def __init__(self, *args, **kwargs):
            pass

    real = cache_utils.Cache
    cache_utils.Cache = _PlainCache
    try:
        spec = importlib.util.spec_from_file_location("alignedkv_reference_KVCache_AlignedKV", path)
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
    finally:
        cache_utils.Cache = real
    return mod.QuantizedCache_AlignedKV
