"""numpy front-end of the CPU oracle (oracle/akv_oracle.c).  TEST INFRASTRUCTURE ONLY.

Only tests, the smoke check and the bench's CPU-baseline leg may import this module; the product package
(alignedkv_b200) never does.  Each function takes numpy byte arrays laid out exactly like the reference's
tensors (extension/k_cache_file.py:45-53, extension/v_cache_file.py:46-54) and the reference op's scalar
arguments (extension/csrc/KV_cache_ops.cpp:5-67), and returns what the reference op returns plus the plane-read
decision codes the reference never materialises (0 = read mid+last, 1 = skip last, 2 = skip mid+last).
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libakv_oracle.so")
_lib = None


def build(force: bool = False) -> str:
    src = os.path.join(_HERE, "akv_oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "-B", "libakv_oracle.so"], check=True, capture_output=True)
    return _LIB_PATH


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        build()
        L = ctypes.CDLL(_LIB_PATH)
        vp, i32, f32 = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
        L.akvo_f64_to_f16.restype = ctypes.c_uint16
        L.akvo_f64_to_f16.argtypes = [ctypes.c_double]
        L.akvo_f16_to_f64.restype = ctypes.c_double
        L.akvo_f16_to_f64.argtypes = [ctypes.c_uint16]
        L.akvo_hfma.restype = ctypes.c_uint16
        L.akvo_hfma.argtypes = [ctypes.c_uint16] * 3
        L.akvo_hmul.restype = ctypes.c_uint16
        L.akvo_hmul.argtypes = [ctypes.c_uint16] * 2
        L.akvo_k_cache_save.restype = None
        L.akvo_k_cache_save.argtypes = [vp] * 4 + [i32] * 8
        L.akvo_k_cache_compute.restype = None
        L.akvo_k_cache_compute.argtypes = [vp] * 8 + [i32] * 6 + [f32, i32]
        L.akvo_v_cache_save.restype = None
        L.akvo_v_cache_save.argtypes = [vp] * 4 + [i32] * 7
        L.akvo_v_cache_test_compute.restype = None
        L.akvo_v_cache_test_compute.argtypes = [vp] * 4 + [i32] * 5
        L.akvo_v_cache_compute.restype = None
        L.akvo_v_cache_compute.argtypes = [vp] * 7 + [i32] * 7
        _lib = L
    return _lib


def _p(a: np.ndarray | None):
    if a is None:
        return None
    assert a.flags["C_CONTIGUOUS"], "oracle arrays must be contiguous"
    return a.ctypes.data_as(ctypes.c_void_p)


def _u8(a: np.ndarray) -> np.ndarray:
    a = np.ascontiguousarray(a)
    return a.view(np.uint8)


def hfma(a: int, b: int, c: int) -> int:
    return int(lib().akvo_hfma(a, b, c))


def hmul(a: int, b: int) -> int:
    return int(lib().akvo_hmul(a, b))


def f64_to_f16_bits(x: float) -> int:
    return int(lib().akvo_f64_to_f16(float(x)))


def f16_bits_to_f64(h: int) -> float:
    return float(lib().akvo_f16_to_f64(int(h)))


def k_cache_save(first8, mid4, last4, k_new_u8, bsz, n_kv_heads, n_blocks, n_max_blocks, d_head, d_block,
                 start_pos, seqlen) -> None:
    """In-place plane write; argument order of KV_cache_ops.cpp:5-16."""
    for a in (first8, mid4, last4):
        assert a.dtype == np.uint8 and a.flags["C_CONTIGUOUS"] and a.flags["WRITEABLE"]
    k_new_u8 = _u8(k_new_u8)
    lib().akvo_k_cache_save(_p(first8), _p(mid4), _p(last4), _p(k_new_u8), bsz, n_kv_heads, n_blocks, n_max_blocks,
                            d_head, d_block, start_pos, seqlen)


def k_cache_compute(first8, mid4, last4, kq_u8, kqmax_u8, q_u8, bsz, n_kv_heads, n_blocks, n_max_blocks, d_head,
                    d_block, seqlen, sqrt_dim, reference):
    """Returns (s_u8 [B,H,1,(n_blocks+1)*d_block*2], codes [B,H,D]); argument order of KV_cache_ops.cpp:18-32.
    The part of s the reference leaves uninitialised ([..., n_blocks*d_block:]) is zero here."""
    s = np.zeros((bsz, n_kv_heads, 1, (n_blocks + 1) * d_block), dtype=np.uint16)
    codes = np.zeros((bsz, n_kv_heads, d_head), dtype=np.uint8)
    kq_u8, kqmax_u8, q_u8 = _u8(kq_u8), _u8(kqmax_u8), _u8(q_u8)
    if n_blocks > 0:
        lib().akvo_k_cache_compute(_p(first8), _p(mid4), _p(last4), _p(kq_u8), _p(kqmax_u8), _p(q_u8), _p(s),
                                   _p(codes), bsz, n_kv_heads, n_blocks, n_max_blocks, d_head, d_block,
                                   float(sqrt_dim), int(bool(reference)))
    return s.view(np.uint8), codes


def v_cache_save(first8, mid4, last4, v_new_u8, bsz, n_local_kv_heads, max_seq_len, head_dim, start_pos,
                 seq_len) -> None:
    """In-place plane write; argument order of KV_cache_ops.cpp:34-43.  v_new_u8 is [B,S,H,2*D]."""
    v_new_u8 = _u8(v_new_u8)
    lib().akvo_v_cache_save(_p(first8), _p(mid4), _p(last4), _p(v_new_u8), bsz, n_local_kv_heads, max_seq_len,
                            head_dim, start_pos, seq_len, int(v_new_u8.shape[1]))


def v_cache_test_compute(first8, mid4, last4, test_s_value_u8, test_s_index_u8, bsz, n_local_kv_heads, max_seq_len,
                         head_dim, top_max_k):
    """Returns u8 [B,H,1,2*D] (fp16 bytes); argument order of KV_cache_ops.cpp:45-54."""
    out = np.zeros((bsz, n_local_kv_heads, 1, head_dim), dtype=np.uint16)
    sv, si = _u8(test_s_value_u8), _u8(test_s_index_u8)
    rows = si.view(np.int32).reshape(-1, top_max_k).astype(np.int64) * top_max_k + np.arange(top_max_k)
    assert rows.min() >= 0 and rows.max() < max_seq_len, "probe row out of range"
    lib().akvo_v_cache_test_compute(_p(first8), _p(sv), _p(si), _p(out), bsz, n_local_kv_heads, max_seq_len,
                                    head_dim, top_max_k)
    return out.view(np.uint8)


def v_cache_compute(first8, mid4, last4, s_u8, amin_u8, bsz, n_local_kv_heads, max_seq_len, head_dim, s_last_dim,
                    start_pos_add_seqlen, reference):
    """Returns (o_u8 [B,H,1,2*D], codes [B,H,n]); argument order of KV_cache_ops.cpp:56-67.
    s_u8 holds fp16 bytes whose (b,h) rows start every s_last_dim halves; amin_u8 is read flat at b*H+h."""
    o = np.zeros((bsz, n_local_kv_heads, 1, head_dim), dtype=np.uint16)
    n = int(start_pos_add_seqlen)
    codes = np.zeros((bsz, n_local_kv_heads, max(n, 1)), dtype=np.uint8)
    s_u8, amin_u8 = _u8(s_u8), _u8(amin_u8)
    assert s_u8.size >= 2 * ((bsz * n_local_kv_heads - 1) * s_last_dim + n)
    assert amin_u8.size >= bsz * n_local_kv_heads
    lib().akvo_v_cache_compute(_p(first8), _p(mid4), _p(last4), _p(s_u8), _p(amin_u8), _p(o), _p(codes), bsz,
                               n_local_kv_heads, max_seq_len, head_dim, s_last_dim, n, int(bool(reference)))
    return o.view(np.uint8), codes[:, :, :n]
