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
