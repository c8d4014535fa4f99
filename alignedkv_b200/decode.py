"""`DecodeLayer`: one layer's AlignedKV cache driven through the one-call decode step of the C ABI.

State and arithmetic are those of the reference's K_Cache_Class / V_Cache_Class pair (extension/k_cache_file.py,
extension/v_cache_file.py) plus the decode branch of QuantizedCache_AlignedKV (model/KVCache_AlignedKV.py:116-124);
the difference is mechanical: the ~35 small tensor operations the reference wrappers run per step are folded into
kernels behind `akv_decode_step`, so a step is a single library call.
"""
from __future__ import annotations

import ctypes
import math

import torch

from . import _lib
from .extension._planes import cdiv, column_block, exponent_field
from .extension.KV_cache_cpp_extention import cuda_module

__all__ = ["DecodeLayer"]


AKV_STEP_REFERENCE, AKV_STEP_ORDER_FREE, AKV_STEP_NO_APPEND, AKV_STEP_TRACK_MAXIMA = 1, 2, 4, 8


class DecodeLayer:
    """One layer's planes, residual buffers and exponent maxima, driven by `akv_decode_step_ex`.

    n_heads is the number of KV heads; n_q_heads (default: the same) may be a multiple of it (grouped-query
    attention; query head i reads KV head i // group).  v_mode "exact" runs P.V in the reference's token order
    (bit-identical to its kernel), "order_free" splits the token axis and accumulates in fp32."""
    def __init__(self, bsz: int, max_seq_len: int, n_heads: int, head_dim: int, device, n_q_heads: int | None = None,
                 v_mode: str = "exact"):
        self.lib = _lib.load()
        self.B, self.L, self.H, self.D = bsz, max_seq_len, n_heads, head_dim
        self.Hq = n_heads if n_q_heads is None else n_q_heads
        if self.Hq % n_heads:
            raise ValueError("n_q_heads must be a multiple of n_heads")
        self.G = self.Hq // n_heads
        if v_mode not in ("exact", "order_free"):
            raise ValueError("v_mode must be 'exact' or 'order_free'")
        self.v_mode = v_mode
        self.device = torch.device(device)
        nmb = cdiv(max_seq_len, column_block)
        z = lambda *shape: torch.zeros(shape, dtype=torch.uint8, device=self.device)  # noqa: E731
        self.k_first_8 = z(bsz, n_heads, nmb, head_dim, column_block)
        self.k_mid_4 = z(bsz, n_heads, nmb, head_dim, column_block // 2)
        self.k_last_4 = z(bsz, n_heads, nmb, head_dim, column_block // 2)
        self.v_first_8 = z(bsz, n_heads, max_seq_len, head_dim)
        self.v_mid_4 = z(bsz, n_heads, max_seq_len, head_dim // 2)
        self.v_last_4 = z(bsz, n_heads, max_seq_len, head_dim // 2)
        self.k_exp_max = z(bsz, 1, n_heads, head_dim)
        self.v_exp_max = z(bsz, 1, n_heads, head_dim)
        self.restk = torch.zeros((bsz, column_block, n_heads, head_dim), dtype=torch.half, device=self.device)
        self.restv = torch.zeros_like(self.restk)
        self.rest_len = 0
        self.rest_start = 0
        self.cache_len = 0
        self.reference = False
        nbytes = self.lib.akv_decode_scratch_bytes_ex(bsz, n_heads, self.G, head_dim, max_seq_len, self._flags())
        if nbytes < 0:
            raise ValueError("bad extents")
        self.scratch = torch.empty(nbytes, dtype=torch.uint8, device=self.device)
        self._sm_count = torch.cuda.get_device_properties(self.device).multi_processor_count
        self._static_ptrs = None
        self.launches = 0

    @property
    def launches(self) -> int:
        """Kernels the library has launched (process-wide) since the counter was last set; `layer.launches = 0`
        resets it.  The count comes from the library's own launch sites, not from arithmetic on this side."""
        return int(self.lib.akv_launch_count()) - self._launch_base

    @launches.setter
    def launches(self, value: int) -> None:
        self._launch_base = int(self.lib.akv_launch_count()) - int(value)

    def _flags(self, append: bool = True) -> int:
        return (AKV_STEP_REFERENCE if getattr(self, "reference", False) else 0) | \
               (AKV_STEP_ORDER_FREE if self.v_mode == "order_free" else 0) | (0 if append else AKV_STEP_NO_APPEND)

    # ------------------------------------------------------------------ prompt
    def prefill(self, k: torch.Tensor, v: torch.Tensor) -> None:
        """Ingest a prompt [B,S,H,D]: whole 64-token blocks to the planes, the tail to the residual buffers, the
        exponent of the signed per-channel maximum to the exponent tensors (extension/k_cache_file.py:76-96,
        extension/v_cache_file.py:79-96) - one pass over the inputs (`akv_prefill`)."""
        B, H, D = self.B, self.H, self.D
        S = k.shape[1]
        assert self.cache_len == 0 and k.shape == (B, S, H, D) and v.shape == (B, S, H, D) and S <= self.L
        for name, t in (("k", k), ("v", v)):
            if t.dtype != torch.half or not t.is_cuda or not t.is_contiguous():
                raise RuntimeError(f"{name}: expected a contiguous CUDA fp16 tensor")
        full = S - S % column_block
        if S > 0 and D % 32 == 0 and D <= 256:
            nbytes = self.lib.akv_prefill_scratch_bytes(B, H, D, S)
            ws = torch.empty(nbytes, dtype=torch.uint8, device=self.device)
            with torch.cuda.device(self.device):
                rc = self.lib.akv_prefill(
                    self.k_first_8.data_ptr(), self.k_mid_4.data_ptr(), self.k_last_4.data_ptr(),
                    self.v_first_8.data_ptr(), self.v_mid_4.data_ptr(), self.v_last_4.data_ptr(),
                    self.k_exp_max.data_ptr(), self.v_exp_max.data_ptr(), self.restk.data_ptr(), self.restv.data_ptr(),
                    k.data_ptr(), v.data_ptr(), ws.data_ptr(), nbytes, B, H, D, self.L, S,
                    torch.cuda.current_stream(self.device).cuda_stream)
            _lib.check("prefill", rc)
        elif S > 0:
            # head sizes the fused kernel does not cover: the operator-by-operator route
            self.k_exp_max.copy_(exponent_field(torch.max(k, dim=1, keepdim=True).values))
            self.v_exp_max.copy_(exponent_field(torch.max(v, dim=1, keepdim=True).values))
            cuda_module.k_cache_save(self.k_first_8, self.k_mid_4, self.k_last_4, k.view(torch.uint8), B, H,
                                     S // column_block, cdiv(self.L, column_block), D, column_block, 0, S)
            cuda_module.v_cache_save(self.v_first_8, self.v_mid_4, self.v_last_4, v.view(torch.uint8), B, H, self.L, D,
                                     0, full)
            self.restk[:, :S - full] = k[:, full:]
            self.restv[:, :S - full] = v[:, full:]
        self.rest_len = S % column_block
        self.rest_start = full
        self.cache_len = S

    # ------------------------------------------------------------------ one decode token
    def decode(self, q: torch.Tensor, k: torch.Tensor | None = None, v: torch.Tensor | None = None, *,
               append: bool = True, packed: bool = False, out: torch.Tensor | None = None,
               mask: torch.Tensor | None = None, exchange=None):
        """Append (k, v) of one token per sequence and return the attention output [B,1,Hq,D] (fp16; written into
        `out` when given).

        append=False leaves the cache as it is (the token belongs to another shard of the sequence).  packed=True
        returns instead the fp32 record [B*Hq, D+2] = (max score, sum of exponentials, output) over this cache's
        tokens, which `akv_lse_merge` combines across the shards of a sequence.

        mask: the additive attention mask of the reference's caller (model/KVCache_AlignedKV.py:119-120), an fp16 CUDA
        tensor of shape [B,1,1,n] or [1,1,1,n] with n >= the cache length after this step (one row per batch row,
        broadcast over the heads); it is added to the fp16 scores in fp16 before the fp32 softmax.

        exchange: the ranks' exchange buffers (`sharded.PeerExchange`) when this layer holds one shard of a sequence:
        the step's last kernel then stores the packed record into every rank's buffer, waits for the others' and the
        call returns the MERGED attention output [B,1,Hq,D], the same on every rank (`akv_decode_step_exchange`)."""
        if exchange is not None and (packed or mask is not None):
            raise RuntimeError("exchange: not together with packed or mask")
        packed = packed or exchange is not None
        B, H, Hq, D = self.B, self.H, self.Hq, self.D
        mask_ptr, mask_stride = None, 0
        if mask is not None:
            need = self.cache_len + (1 if append else 0)
            if mask.dtype != torch.half or not mask.is_cuda or mask.dim() != 4 or mask.shape[1] != 1 or \
                    mask.shape[2] != 1 or mask.shape[0] not in (1, B) or mask.shape[3] < need or mask.stride(3) != 1:
                raise RuntimeError(f"mask: expected a CUDA fp16 tensor of shape [{B} or 1, 1, 1, >= {need}] with a "
                                   "unit stride along the positions")
            mask_ptr, mask_stride = mask.data_ptr(), (mask.stride(0) if mask.shape[0] == B else 0)
        checks = [("q", q, Hq)] + ([("k", k, H), ("v", v, H)] if append else [])
        for name, t, heads in checks:
            if t is None or t.shape != (B, 1, heads, D) or t.dtype != torch.half or not t.is_cuda or \
                    not t.is_contiguous():
                raise RuntimeError(f"{name}: expected a contiguous CUDA fp16 tensor of shape {(B, 1, heads, D)}")
        if append and self.cache_len + 1 > self.L:
            raise RuntimeError(f"cache is full ({self.L} tokens)")
        if out is not None and (packed or out.shape != (B, 1, Hq, D) or out.dtype != torch.half or not out.is_cuda or
                                not out.is_contiguous()):
            raise RuntimeError(f"out: expected a contiguous CUDA fp16 tensor of shape {(B, 1, Hq, D)}")
        if out is None and not packed:
            out = torch.empty((B, 1, Hq, D), dtype=torch.half, device=self.device)
        rec = torch.empty((B * Hq, D + 2), dtype=torch.float32, device=self.device) if packed else None
        # (the planes, exponent maxima, residual buffers and the workspace never move: their addresses are taken once;
        # the device is only switched when it is not the current one - both keep the host's share of a step small,
        # which is what bounds a rank whose CPU is slow)
        ptrs = self._static_ptrs
        if ptrs is None:
            ptrs = self._static_ptrs = tuple(t.data_ptr() for t in (
                self.k_first_8, self.k_mid_4, self.k_last_4, self.v_first_8, self.v_mid_4, self.v_last_4,
                self.k_exp_max, self.v_exp_max, self.restk, self.restv)) + (self.scratch.data_ptr(), self.scratch.numel())
        args = ptrs[:10] + (
            q.data_ptr(), k.data_ptr() if append else None, v.data_ptr() if append else None,
            out.data_ptr() if out is not None else None, rec.data_ptr() if rec is not None else None,
            mask_ptr, mask_stride, ptrs[10], ptrs[11], B, H, self.G, D, self.L, self.rest_len, self.rest_start,
            self._flags(append), torch.cuda.current_stream(self.device).cuda_stream)
        fn = self.lib.akv_decode_step_masked
        if exchange is not None:
            out = torch.empty((B, 1, Hq, D), dtype=torch.half, device=self.device)
            fn = self.lib.akv_decode_step_exchange
            args = args[:13] + (out.data_ptr(),) + args[14:15] + args[17:27] + (
                exchange.bufs, exchange.rank, exchange.world, exchange.next_epoch(), exchange.timeout_ms, args[27])
        if torch.cuda.current_device() == self.device.index:
            rc = fn(*args)
        else:
            with torch.cuda.device(self.device):
                rc = fn(*args)
        _lib.check("decode_step", rc)
        self.last_q = q                                   # (for bytes_accounting)
        flush = append and self.rest_len + 1 == column_block
        qn = self.rest_start + (column_block if flush else 0)
        rest = 0 if flush else self.rest_len + (1 if append else 0)
        self.rest_len, self.rest_start = rest, qn
        if append:
            self.cache_len += 1
        return out if exchange is not None else (rec if packed else out)

    # ------------------------------------------------------------------ benchmark helpers
    def snapshot(self):
        """What is needed to come back to the current length later (`restore`): the counters and the exponent maxima."""
        return dict(rest_len=self.rest_len, rest_start=self.rest_start, cache_len=self.cache_len,
                    k_exp=self.k_exp_max.clone(), v_exp=self.v_exp_max.clone())

    def restore(self, snap) -> None:
        """Roll the cache back to a snapshot (`akv_rollback`): the exponent maxima are put back and the K nibble planes
        of blocks written since are cleared, because the K writer accumulates nibbles
        (extension/csrc/K_cache.cu:52-56).  Tokens that were still in the residual buffer at the snapshot stay
        there: later appends only wrote rows behind them."""
        first_blk = snap["rest_start"] // column_block
        last_blk = self.rest_start // column_block
        appended = self.cache_len - snap["cache_len"]
        if appended < 0 or (snap["rest_len"] and snap["rest_len"] + appended > column_block):
            raise RuntimeError("restore: the residual tokens of the snapshot have been overwritten since")
        with torch.cuda.device(self.device):
            rc = self.lib.akv_rollback(self.k_mid_4.data_ptr(), self.k_last_4.data_ptr(), self.k_exp_max.data_ptr(),
                                       self.v_exp_max.data_ptr(), snap["k_exp"].data_ptr(), snap["v_exp"].data_ptr(),
                                       self.B, self.H, self.D, self.L, first_blk, max(0, last_blk - first_blk),
                                       torch.cuda.current_stream(self.device).cuda_stream)
        _lib.check("rollback", rc)
        self.rest_len, self.rest_start, self.cache_len = snap["rest_len"], snap["rest_start"], snap["cache_len"]

    def reset_counters(self) -> None:
        self.launches = 0
        self.lib.akv_set_tuning(b"timing", 1)
        self.lib.akv_timing_reset()

    def kernel_times(self):
        """Median CUDA-event duration of the two streaming kernels over the steps since reset_counters()."""
        torch.cuda.synchronize(self.device)
        k_us, v_us = ctypes.c_double(0), ctypes.c_double(0)
        n = self.lib.akv_timing_read(ctypes.byref(k_us), ctypes.byref(v_us))
        self.lib.akv_set_tuning(b"timing", 0)
        if n == 0:
            return {}
        return {"k_compute": {"us": k_us.value, "launches": n}, "v_compute": {"us": v_us.value, "launches": n}}

    def bytes_accounting(self, q: torch.Tensor | None = None):
        """Algorithmic plane bytes of the LAST decode step under its read decisions (mid plane iff code < 2, low
        plane iff code < 1), from the state the step left behind, plus the dense fp16 equivalent."""
        B, H, Hq, G, D = self.B, self.H, self.Hq, self.G, self.D
        q = self.last_q if q is None else q
        qn = self.rest_start
        # K: per (batch, KV head, channel) the union over the group's query heads of the plane reads
        kq = exponent_field(q).view(B, 1, H, G, D) + self.k_exp_max.view(B, 1, H, 1, D)
        diff = (kq.max(dim=4, keepdim=True).values - kq)
        k_rows = float(B * H * D) + 0.5 * float((diff < 8).any(dim=3).sum()) + 0.5 * float((diff < 4).any(dim=3).sum())
        k_bytes = qn * k_rows
        R = (qn // column_block + 1) * column_block
        p = self.scratch[:B * Hq * R * 2].view(torch.half).view(B, Hq, R)[..., :qn]
        amin_off = self._scratch_offset("amin")
        amin = self.scratch[amin_off:amin_off + B * Hq].to(torch.int32).view(B, Hq, 1)
        d = ((((amin << 10) & 0xFFFF) - p.view(torch.int16).to(torch.int32)) << 16) >> 16
        d = d.view(B, H, G, qn)
        v_rows = float(B * H * qn) + 0.5 * float((d < 0x800).any(dim=2).sum()) + 0.5 * float((d < 0x400).any(dim=2).sum())
        v_bytes = D * v_rows
        rest = 4.0 * (self.cache_len - qn) * D * B * H
        dense = 4.0 * B * H * self.cache_len * D
        return {"k_compute": k_bytes, "v_compute": v_bytes, "read": k_bytes + v_bytes + rest, "dense": dense}

    def _scratch_offset(self, name: str) -> int:
        B, H, D = self.B, self.Hq, self.D
        R = (cdiv(self.L, column_block) + 1) * column_block
        up = lambda x: (x + 255) & ~255  # noqa: E731
        sizes = [("s", B * H * R * 2), ("kq", B * H * D), ("kqmax", B * H), ("pval", B * H * 32 * 2),
                 ("pidx", B * H * 32 * 4), ("test_o", B * H * D * 2), ("amin", B * H), ("o_main", B * H * D * 2)]
        off = 0
        for n, sz in sizes:
            if n == name:
                return off
            off += up(sz)
        raise KeyError(name)
