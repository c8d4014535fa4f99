"""`K_Cache_Class`: per-layer K plane store with the reference's surface (extension/k_cache_file.py:13-159).

Same constructor, attributes (`k_cache_first_8`, `k_cache_mid_4`, `k_cache_last_4`, `k_cache_exp_column_max`,
`restk`, `restklen`, `reststartpos`, `current_cache_len`) and methods (`save`, `decoding_compute`, `zerolize`).
The plane writer and the aligned q.K^T run in the sm_100a library through `cuda_module`.

Not reproduced: the debugging `print` the reference emits on every prefill (extension/k_cache_file.py:91).
"""
from __future__ import annotations

import math

import torch

from ._planes import ResidualBuffer, bits_in_a_channel, cdiv, column_block, exponent_field
from .KV_cache_cpp_extention import cuda_module

__all__ = ["K_Cache_Class", "bits_in_a_channel", "column_block", "cdiv"]


class K_Cache_Class(torch.nn.Module):
    def __init__(self, bsz: int, max_seq_len: int, n_local_kv_heads: int, head_dim: int, layer_idx: int,
                 device: str | torch.device = "cuda:0", register_buffer: bool = False):
        super().__init__()
        self.bsz = bsz
        self.max_seq_len = max_seq_len
        self.n_local_kv_heads = n_local_kv_heads
        self.head_dim = head_dim
        self.n_max_blocks = cdiv(max_seq_len, column_block)
        self.device = device
        # token-minor layout: [bsz, heads, block, channel, token-in-block] (extension/k_cache_file.py:45-53)
        shapes = {
            "k_cache_first_8": (bsz, n_local_kv_heads, self.n_max_blocks, head_dim, column_block),
            "k_cache_mid_4": (bsz, n_local_kv_heads, self.n_max_blocks, head_dim, column_block // 2),
            "k_cache_last_4": (bsz, n_local_kv_heads, self.n_max_blocks, head_dim, column_block // 2),
            "k_cache_exp_column_max": (bsz, 1, n_local_kv_heads, head_dim),
        }
        for name, shape in shapes.items():
            t = torch.zeros(shape, dtype=torch.uint8, device=device)
            if register_buffer:  # static addresses for torch.compile callers (extension/k_cache_file.py:24-43)
                self.register_buffer(f"{name}_layer_{layer_idx}", t)
                t = getattr(self, f"{name}_layer_{layer_idx}")
                torch._dynamo.mark_static_address(t)
            setattr(self, name, t)
        self._rest = ResidualBuffer(bsz, n_local_kv_heads, head_dim, device)
        self.current_cache_len = 0

    # ---- the reference's attribute names for the residual buffer
    @property
    def restk(self):
        return self._rest.data

    @restk.setter
    def restk(self, value):
        self._rest.data = value

    @property
    def restklen(self) -> int:
        return self._rest.fill

    @restklen.setter
    def restklen(self, value: int):
        self._rest.fill = value

    @property
    def reststartpos(self) -> int:
        return self._rest.start

    @reststartpos.setter
    def reststartpos(self, value: int):
        self._rest.start = value

    def zerolize(self):
        """Clear planes and exponent maxima (required before reuse: nibbles are accumulated, not stored)."""
        for t in (self.k_cache_first_8, self.k_cache_mid_4, self.k_cache_last_4, self.k_cache_exp_column_max):
            t.zero_()
        self.current_cache_len = 0

    def _write_blocks(self, tokens: torch.Tensor, n_blocks: int, start_pos: int, seqlen: int) -> None:
        cuda_module.k_cache_save(self.k_cache_first_8, self.k_cache_mid_4, self.k_cache_last_4,
                                 tokens.view(torch.uint8), self.bsz, self.n_local_kv_heads, n_blocks,
                                 self.n_max_blocks, self.head_dim, column_block, start_pos, seqlen)

    def save(self, new_k: torch.Tensor, start_pos: int, seqlen: int):
        """Prefill (start_pos == 0) or single-token append (extension/k_cache_file.py:69-118)."""
        want = (self.bsz, seqlen, self.n_local_kv_heads, self.head_dim)
        assert new_k.shape == want, f"new_k.shape: {new_k.shape} != {want}"
        assert start_pos + seqlen <= self.max_seq_len, f"start_pos + seqlen: {start_pos + seqlen} > {self.max_seq_len}"
        assert start_pos == 0 or seqlen == 1, f"start_pos: {start_pos}, seqlen: {seqlen}"
        assert start_pos == self.current_cache_len, "start pos != current KV-Cache len"
        self.current_cache_len += seqlen
        if start_pos == 0:
            # exponent of the SIGNED per-channel maximum over the prompt (extension/k_cache_file.py:77-78)
            self.k_cache_exp_column_max = exponent_field(torch.max(new_k, dim=1, keepdim=True).values)
            self._write_blocks(new_k, seqlen // column_block, start_pos, seqlen)
            self._rest.load_tail(new_k, seqlen)
        else:
            self.k_cache_exp_column_max = torch.maximum(self.k_cache_exp_column_max, exponent_field(new_k))
            if self._rest.push(new_k, seqlen):
                self._write_blocks(self._rest.data, 1, self._rest.start, column_block)
                self._rest.advance()

    def decoding_compute(self, q: torch.Tensor, start_pos: int, seqlen: int, reference: bool = False):
        """Scores of one decode token against the whole cache, fp16 [bsz, heads, 1, (n_blocks+1)*64], -inf past
        the last cached token (extension/k_cache_file.py:132-159)."""
        assert q.shape[2] == self.n_local_kv_heads, "we currently only support MHA, don't support GQA"
        want = (self.bsz, seqlen, self.n_local_kv_heads, self.head_dim)
        assert q.shape == want, f"q.shape: {q.shape} != {want}"
        # alignment inputs: exponent upper bound of every product q_d * k_{t,d}, and its maximum over channels
        k_column_max_multiply_q = exponent_field(q) + self.k_cache_exp_column_max
        k_column_max_multiply_q_max = torch.max(k_column_max_multiply_q, dim=3, keepdim=True).values
        inv_sqrt_d = 1.0 / math.sqrt(self.head_dim)
        s = cuda_module.k_cache_compute(self.k_cache_first_8, self.k_cache_mid_4, self.k_cache_last_4,
                                        k_column_max_multiply_q, k_column_max_multiply_q_max, q.view(torch.uint8),
                                        self.bsz, self.n_local_kv_heads, self._rest.start // column_block,
                                        self.n_max_blocks, self.head_dim, column_block, self._rest.start,
                                        inv_sqrt_d, reference).view(torch.half)
        assert self._rest.fill + self._rest.start == start_pos + seqlen
        # tokens still in the fp16 residual buffer: plain dot products
        rest_kt = self._rest.data.transpose(1, 2).transpose(2, 3)[:, :, :, :self._rest.fill]
        s[:, :, :, self._rest.start:self._rest.start + self._rest.fill] = \
            torch.matmul(q.transpose(1, 2), rest_kt) / math.sqrt(self.head_dim)
        s[:, :, :, start_pos + seqlen:] = float("-inf")
        return s
