"""Shared input generators and small adapters for the tests (seeded, BASELINE-shaped distributions)."""
from __future__ import annotations

import importlib.util
import os

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
OUTLIER_CHANNELS = (3, 34, 65, 96)


def make_kvq(seed: int, B: int, L: int, H: int, D: int, outliers: bool = True):
    """K, V [B,L,H,D] and q [B,1,H,D] as float16: N(0,1) drawn in fp32; 4 K channels per head scaled x20."""
    rng = np.random.default_rng(seed)
    k = rng.standard_normal((B, L, H, D), dtype=np.float32)
    v = rng.standard_normal((B, L, H, D), dtype=np.float32)
    q = rng.standard_normal((B, 1, H, D), dtype=np.float32)
    if outliers:
        for c in OUTLIER_CHANNELS:
            if c < D:
                k[..., c] *= 20.0
    return k.astype(np.float16), v.astype(np.float16), q.astype(np.float16)


def exponent_field(x16: np.ndarray) -> np.ndarray:
    return ((x16.view(np.uint16) >> 10) & 0x1F).astype(np.uint8)


def k_planes_np(B, H, nmb, D, d_block=64):
    return (np.zeros((B, H, nmb, D, d_block), np.uint8), np.zeros((B, H, nmb, D, d_block // 2), np.uint8),
            np.zeros((B, H, nmb, D, d_block // 2), np.uint8))


def v_planes_np(B, H, max_seq_len, D):
    return (np.zeros((B, H, max_seq_len, D), np.uint8), np.zeros((B, H, max_seq_len, D // 2), np.uint8),
            np.zeros((B, H, max_seq_len, D // 2), np.uint8))


def softmax_probs(seed: int, B: int, H: int, n: int, pad: int = 0, peaky: float = 4.0) -> np.ndarray:
    """fp16 probabilities [B,H,1,n+pad] (pad entries are 0), from fp32 softmax of scaled normal scores."""
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((B, H, 1, n), dtype=np.float32) * peaky
    e = np.exp(x - x.max(-1, keepdims=True))
    p = (e / e.sum(-1, keepdims=True)).astype(np.float16)
    if pad:
        p = np.concatenate([p, np.zeros((B, H, 1, pad), np.float16)], -1)
    return np.ascontiguousarray(p)


def load_reference_extension():
    """The unmodified reference extension compiled for sm_100a (oracle/_ref), or None when it was not built."""
    so = os.path.join(ROOT, "oracle", "_ref", "kv_cache_cuda.so")
    if not os.path.exists(so):
        return None
    import torch  # noqa: F401  (the extension links against libtorch)
    spec = importlib.util.spec_from_file_location("kv_cache_cuda", so)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def reference_root():
    """A checkout of the reference: $AKV_REFERENCE_ROOT, else the vendored copy under baseline/_ref (git-ignored; made
    by oracle/build_ref.py), else a sibling directory `reference` next to this repository.  None when there is none."""
    for cand in (os.environ.get("AKV_REFERENCE_ROOT"), os.path.join(ROOT, "baseline", "_ref"),
                 os.path.join(os.path.dirname(ROOT), "reference")):
        if cand and os.path.exists(os.path.join(cand, "model", "KVCache_AlignedKV.py")):
            return cand
    return None


def load_reference_caller():
    """The reference's own QuantizedCache_AlignedKV (model/KVCache_AlignedKV.py, unchanged) running on this package's
    operators, or None when no reference checkout is at hand."""
    root = reference_root()
    if root is None:
        return None
    import alignedkv_b200
    return alignedkv_b200.load_reference_cache(root)


class CudaModuleSpy:
    """Forwards every operator call to a real `cuda_module` and keeps the last arguments and result of each, so that a
    test can read the tensors the reference's wrappers exchange with its kernels (scores, probabilities, thresholds)."""

    def __init__(self, real):
        self._real = real
        self.calls = {}

    def __getattr__(self, name):
        fn = getattr(self._real, name)

        def wrapped(*args):
            out = fn(*args)
            self.calls[name] = {"args": args, "out": out}
            return out

        return wrapped


def load_reference_stack():
    """The COMPLETE reference on this machine's GPU: its caller (model/KVCache_AlignedKV.py), its wrapper classes
    (extension/k_cache_file.py, extension/v_cache_file.py) - all imported unchanged from the vendored checkout - over
    its own CUDA kernels compiled unmodified for sm_100a (oracle/_ref/kv_cache_cuda.so).  Returns
    (QuantizedCache_AlignedKV, spy) or None when the checkout or the compiled extension is missing.  The reference's
    loader module (extension/KV_cache_cpp_extention.py, which compiles at import time with a hard-coded host compiler)
    is the one thing replaced: a stub module whose `cuda_module` is the spy around the compiled extension."""
    import sys
    import types
    root, ext = reference_root(), load_reference_extension()
    if root is None or ext is None:
        return None
    import transformers.cache_utils as cache_utils
    spy = CudaModuleSpy(ext)
    names = ["extension", "extension.KV_cache_cpp_extention", "extension.k_cache_file", "extension.v_cache_file"]
    saved = {n: sys.modules.get(n) for n in names}
    pkg = types.ModuleType("extension")
    pkg.__path__ = [os.path.join(root, "extension")]
    stub = types.ModuleType("extension.KV_cache_cpp_extention")
    stub.cuda_module = spy
    for n in names:
        sys.modules.pop(n, None)
    sys.modules["extension"] = pkg
    sys.modules["extension.KV_cache_cpp_extention"] = stub

    class _PlainCache:
        def __init__(self, *a, **k):
            pass

    real = cache_utils.Cache
    cache_utils.Cache = _PlainCache
    try:
        spec = importlib.util.spec_from_file_location("akv_full_reference_KVCache_AlignedKV",
                                                      os.path.join(root, "model", "KVCache_AlignedKV.py"))
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
    finally:
        cache_utils.Cache = real
        for n in names:
            sys.modules.pop(n, None)
            if saved[n] is not None:
                sys.modules[n] = saved[n]
    return mod.QuantizedCache_AlignedKV, spy
