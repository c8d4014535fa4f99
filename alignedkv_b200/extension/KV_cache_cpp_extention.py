"""`cuda_module`: the five operators of the reference's torch extension, served by libalignedkv_b200.so.

The reference builds its kernels at import time and exposes the pybind module as `cuda_module`
(extension/KV_cache_cpp_extention.py:6-9; operators at extension/csrc/KV_cache_ops.cpp:69-75).  This module
keeps the attribute name and every operator's positional signature; behind it each call goes through ctypes
into the prebuilt C-ABI library and launches on torch's current CUDA stream.

Error behaviour kept from the reference: tensor arguments must be uint8 (`data_ptr<unsigned char>()` throws for
any other dtype, e.g. extension/csrc/K_cache.cu:109-112).  Added: tensors must be contiguous CUDA tensors on
one device, and a failed launch raises instead of being ignored.
"""
from __future__ import annotations

import torch

from .. import _lib

__all__ = ["cuda_module"]


def _u8(name: str, t: torch.Tensor, dev: torch.device | None = None) -> int:
    if not isinstance(t, torch.Tensor):
        raise TypeError(f"{name}: expected a torch.Tensor, got {type(t).__name__}")
    if t.dtype != torch.uint8:
        raise RuntimeError(f"{name}: expected scalar type Byte but found {t.dtype}")
    if not t.is_cuda:
        raise RuntimeError(f"{name}: expected a CUDA tensor (alignedkv_b200 has no CPU path)")
    if dev is not None and t.device != dev:
        raise RuntimeError(f"{name}: tensor is on {t.device}, expected {dev}")
    if not t.is_contiguous():
        raise RuntimeError(f"{name}: tensor must be contiguous")
    return t.data_ptr()


def _stream(dev: torch.device) -> int:
    return torch.cuda.current_stream(dev).cuda_stream


def _cuda_device_of(name: str, t: torch.Tensor) -> torch.device:
    """Device of the tensor that anchors a call (checked before a device context is entered)."""
    _u8(name, t)
    return t.device


class _CudaModule:
    """Stand-in for the pybind module `kv_cache_cuda`."""

    def __init__(self):
        self._lib = _lib.load()

    # KV_cache_ops.cpp:5-16
    def k_cache_save(self, k_cache_first_8, k_cache_mid_4, k_cache_last_4, k_new, bsz, n_kv_heads, n_blocks,
                     n_max_blocks, d_head, d_block, start_pos, seqlen) -> None:
        dev = _cuda_device_of("k_new", k_new)
        with torch.cuda.device(dev):
            rc = self._lib.akv_k_cache_save(
                _u8("k_cache_first_8", k_cache_first_8, dev), _u8("k_cache_mid_4", k_cache_mid_4, dev),
                _u8("k_cache_last_4", k_cache_last_4, dev), _u8("k_new", k_new),
                int(bsz), int(n_kv_heads), int(n_blocks), int(n_max_blocks), int(d_head), int(d_block),
                int(start_pos), int(seqlen), _stream(dev))
        _lib.check("k_cache_save", rc)

    # KV_cache_ops.cpp:18-32
    def k_cache_compute(self, k_cache_first_8, k_cache_mid_4, k_cache_last_4, k_column_max_multiply_q,
                        k_column_max_multiply_q_max, q, bsz, n_kv_heads, n_blocks, n_max_blocks, d_head, d_block,
                        seqlen, sqrt_dim, reference) -> torch.Tensor:
        dev = _cuda_device_of("q", q)
        # same shape and (uninitialised) allocation as extension/csrc/K_cache.cu:329-330
        s = torch.empty((bsz, n_kv_heads, 1, (n_blocks + 1) * d_block * 2), dtype=torch.uint8, device=dev)
        if n_blocks == 0:
            return s
        with torch.cuda.device(dev):
            rc = self._lib.akv_k_cache_compute(
                _u8("k_cache_first_8", k_cache_first_8, dev), _u8("k_cache_mid_4", k_cache_mid_4, dev),
                _u8("k_cache_last_4", k_cache_last_4, dev),
                _u8("k_column_max_multiply_q", k_column_max_multiply_q, dev),
                _u8("k_column_max_multiply_q_max", k_column_max_multiply_q_max, dev), _u8("q", q),
                s.data_ptr(), int(bsz), int(n_kv_heads), int(n_blocks), int(n_max_blocks), int(d_head),
                int(d_block), int(seqlen), float(sqrt_dim), int(bool(reference)), _stream(dev))
        _lib.check("k_cache_compute", rc)
        return s

    # KV_cache_ops.cpp:34-43
    def v_cache_save(self, v_cache_first_8, v_cache_mid_4, v_cache_last_4, v_new, bsz, n_local_kv_heads,
                     max_seq_len, head_dim, start_pos, seq_len) -> None:
        dev = _cuda_device_of("v_new", v_new)
        with torch.cuda.device(dev):
            rc = self._lib.akv_v_cache_save(
                _u8("v_cache_first_8", v_cache_first_8, dev), _u8("v_cache_mid_4", v_cache_mid_4, dev),
                _u8("v_cache_last_4", v_cache_last_4, dev), _u8("v_new", v_new),
                int(bsz), int(n_local_kv_heads), int(max_seq_len), int(head_dim), int(start_pos), int(seq_len),
                int(v_new.size(1)), _stream(dev))
        _lib.check("v_cache_save", rc)

    # KV_cache_ops.cpp:45-54
    def v_cache_test_compute(self, v_cache_first_8, v_cache_mid_4, v_cache_last_4, test_s_value, test_s_index, bsz,
                             n_local_kv_heads, max_seq_len, head_dim, top_max_k) -> torch.Tensor:
        dev = _cuda_device_of("test_s_value", test_s_value)
        test_o = torch.empty((bsz, n_local_kv_heads, 1, head_dim * 2), dtype=torch.uint8, device=dev)
        with torch.cuda.device(dev):
            rc = self._lib.akv_v_cache_test_compute(
                _u8("v_cache_first_8", v_cache_first_8, dev), _u8("v_cache_mid_4", v_cache_mid_4, dev),
                _u8("v_cache_last_4", v_cache_last_4, dev), _u8("test_s_value", test_s_value),
                _u8("test_s_index", test_s_index, dev), test_o.data_ptr(),
                int(bsz), int(n_local_kv_heads), int(max_seq_len), int(head_dim), int(top_max_k), _stream(dev))
        _lib.check("v_cache_test_compute", rc)
        return test_o

    # KV_cache_ops.cpp:56-67
    def v_cache_compute(self, v_cache_first_8, v_cache_mid_4, v_cache_last_4, s, s_exp_expect_alignment_min, bsz,
                        n_local_kv_heads, max_seq_len, head_dim, s_last_dim, start_pos_add_seqlen,
                        reference) -> torch.Tensor:
        dev = _cuda_device_of("v_cache_first_8", v_cache_first_8)
        o = torch.empty((bsz, n_local_kv_heads, 1, head_dim * 2), dtype=torch.uint8, device=dev)
        # `s` may be a sliced view (extension/v_cache_file.py:150,184): like the reference, only its base
        # pointer and the row stride passed as s_last_dim are used, so contiguity is not required here.
        if not isinstance(s, torch.Tensor) or s.dtype != torch.uint8:
            raise RuntimeError(f"s: expected scalar type Byte but found {getattr(s, 'dtype', type(s))}")
        if not s.is_cuda or s.device != dev:
            raise RuntimeError("s: expected a CUDA tensor on the planes' device")
        with torch.cuda.device(dev):
            rc = self._lib.akv_v_cache_compute(
                _u8("v_cache_first_8", v_cache_first_8, dev), _u8("v_cache_mid_4", v_cache_mid_4, dev),
                _u8("v_cache_last_4", v_cache_last_4, dev), s.data_ptr(),
                _u8("s_exp_expect_alignment_min", s_exp_expect_alignment_min, dev), o.data_ptr(),
                int(bsz), int(n_local_kv_heads), int(max_seq_len), int(head_dim), int(s_last_dim),
                int(start_pos_add_seqlen), int(bool(reference)), _stream(dev))
        _lib.check("v_cache_compute", rc)
        return o


cuda_module = _CudaModule()
