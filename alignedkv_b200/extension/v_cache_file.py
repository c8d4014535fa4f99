"""`V_Cache_Class`: per-layer V plane store with the reference's surface (extension/v_cache_file.py:14-190).

Same constructor, attributes (`v_cache_first_8`, `v_cache_mid_4`, `v_cache_last_4`, `v_cache_exp_column_max`,
`restv`, `restvlen`, `reststartpos`, `current_cache_len`, `top_max_k`) and methods (`save`, `test_compute`,
`decoding_compute`, `zerolize`).  Plane writer, magnitude probe and aligned P.V run in the sm_100a library.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from ._planes import ResidualBuffer, bits_in_a_channel, cdiv, column_block, exponent_field
from .KV_cache_cpp_extention import cuda_module

__all__ = ["V_Cache_Class", "bits_in_a_channel", "column_block", "cdiv"]

FP16_EXP_BIAS = 15


class V_Cache_Class(torch.nn.Module):
    def __init__(self, bsz: int, max_seq_len: int, n_local_kv_heads: int, head_dim: int, layer_id: int,
                 device: str | torch.device = "cuda:0", register_buffer: bool = False, top_max_k: int = 32):
        super().__init__()
        self.bsz = bsz
        self.max_seq_len = max_seq_len
        self.n_local_kv_heads = n_local_kv_heads
        self.head_dim = head_dim
        self.n_max_blocks = cdiv(max_seq_len, column_block)
        self.device = device
        self.top_max_k = top_max_k
        # token-major layout: [bsz, heads, token, channel] (extension/v_cache_file.py:46-54)
        shapes = {
            "v_cache_first_8": (bsz, n_local_kv_heads, max_seq_len, head_dim),
            "v_cache_mid_4": (bsz, n_local_kv_heads, max_seq_len, head_dim // 2),
            "v_cache_last_4": (bsz, n_local_kv_heads, max_seq_len, head_dim // 2),
            "v_cache_exp_column_max": (bsz, 1, n_local_kv_heads, head_dim),
        }
        for name, shape in shapes.items():
            t = torch.zeros(shape, dtype=torch.uint8, device=device)
            if register_buffer:
                self.register_buffer(f"{name}_layer_{layer_id}", t)
                t = getattr(self, f"{name}_layer_{layer_id}")
                torch._dynamo.mark_static_address(t)
            setattr(self, name, t)
        self._rest = ResidualBuffer(bsz, n_local_kv_heads, head_dim, device)
        self.current_cache_len = 0

    @property
    def restv(self):
        return self._rest.data

    @restv.setter
    def restv(self, value):
        self._rest.data = value

    @property
    def restvlen(self) -> int:
        return self._rest.fill

    @restvlen.setter
    def restvlen(self, value: int):
        self._rest.fill = value

    @property
    def reststartpos(self) -> int:
        return self._rest.start

    @reststartpos.setter
    def reststartpos(self, value: int):
        self._rest.start = value

    def zerolize(self):
        for t in (self.v_cache_first_8, self.v_cache_mid_4, self.v_cache_last_4, self.v_cache_exp_column_max):
            t.zero_()
        self.current_cache_len = 0

    def _write_tokens(self, tokens: torch.Tensor, start_pos: int, count: int) -> None:
        cuda_module.v_cache_save(self.v_cache_first_8, self.v_cache_mid_4, self.v_cache_last_4,
                                 tokens.view(torch.uint8), self.bsz, self.n_local_kv_heads, self.max_seq_len,
                                 self.head_dim, start_pos, count)

    def save(self, new_v: torch.Tensor, start_pos: int, seqlen: int):
        """Prefill (start_pos == 0) or single-token append (extension/v_cache_file.py:72-116)."""
        want = (self.bsz, seqlen, self.n_local_kv_heads, self.head_dim)
        assert new_v.shape == want, f"new_v.shape: {new_v.shape} != {want}"
        assert start_pos + seqlen <= self.max_seq_len, f"start_pos + seqlen: {start_pos + seqlen} > {self.max_seq_len}"
        assert start_pos == 0 or seqlen == 1, f"start_pos: {start_pos}, seqlen: {seqlen}"
        assert start_pos == self.current_cache_len, "start pos != current KV-Cache len"
        self.current_cache_len += seqlen
        if start_pos == 0:
            self.v_cache_exp_column_max = exponent_field(torch.max(new_v, dim=1, keepdim=True).values)
            self._write_tokens(new_v, start_pos, seqlen - seqlen % column_block)
            self._rest.load_tail(new_v, seqlen)
        else:
            self.v_cache_exp_column_max = torch.maximum(self.v_cache_exp_column_max, exponent_field(new_v))
            if self._rest.push(new_v, seqlen):
                self._write_tokens(self._rest.data, self._rest.start, column_block)
                self._rest.advance()

    def test_compute(self, s: torch.Tensor, start_pos: int, seqlen: int, top_max_k: int):
        """Magnitude probe: for every residue class (token index mod top_max_k) take the largest probability and
        its first position, weigh the |high byte| rows of those tokens, return the exponent bytes of the result
        with the lowest bit cleared (extension/v_cache_file.py:119-143; `& 0x1F - 1` there parses as `& 0x1E`)."""
        if start_pos + seqlen == s.shape[-1]:
            groups = cdiv(start_pos + seqlen, top_max_k)
            s = F.pad(s, (0, groups * top_max_k - start_pos - seqlen), "constant", 0)
        else:
            groups = s.shape[-1] // top_max_k
        s = s.view(self.bsz, self.n_local_kv_heads, groups, top_max_k)
        test_s_value, test_s_index = torch.max(s, dim=2, keepdim=True)
        test_s_index = test_s_index.to(torch.int32)
        test_o = cuda_module.v_cache_test_compute(self.v_cache_first_8, self.v_cache_mid_4, self.v_cache_last_4,
                                                  test_s_value.view(torch.uint8), test_s_index.view(torch.uint8),
                                                  self.bsz, self.n_local_kv_heads, self.max_seq_len, self.head_dim,
                                                  top_max_k).view(torch.half)
        return exponent_field(test_o) & 0x1E

    def decoding_compute(self, s: torch.Tensor, start_pos: int, seqlen: int, reference: bool = False):
        """Attention output of one decode token, fp16 [bsz, heads, 1, head_dim]
        (extension/v_cache_file.py:145-190)."""
        assert s.shape[1] == self.n_local_kv_heads, "we currently only support MHA, don't support GQA"
        want = (self.bsz, self.n_local_kv_heads, 1, s.shape[-1])
        assert s.shape == want, f"s.shape: {s.shape} != {(self.bsz, self.n_local_kv_heads, 1, start_pos + seqlen)}"
        assert start_pos + seqlen <= self.max_seq_len, f"start_pos + seqlen: {start_pos + seqlen} > {self.max_seq_len}"
        assert start_pos == 0 or seqlen == 1, f"start_pos: {start_pos}, seqlen: {seqlen}"
        quantized = self._rest.start
        s_cut = s[:, :, :, :quantized]
        test_o_exp = self.test_compute(s_cut if quantized else s, start_pos, seqlen, self.top_max_k)
        # Smallest probability exponent whose product with this head's largest V can still reach the probe
        # result's precision.  [B,H,1,D] - [B,1,H,D] broadcasts to [B,H,H,D] in uint8 arithmetic, exactly as in
        # the reference (extension/v_cache_file.py:156-160); the kernel reads the result flat at b*H+h.
        s_exp_expect_alignment = test_o_exp + FP16_EXP_BIAS - self.v_cache_exp_column_max
        s_exp_expect_alignment_min = torch.min(s_exp_expect_alignment, dim=-1, keepdim=True).values
        o = cuda_module.v_cache_compute(self.v_cache_first_8, self.v_cache_mid_4, self.v_cache_last_4,
                                        s_cut.view(torch.uint8), s_exp_expect_alignment_min, self.bsz,
                                        self.n_local_kv_heads, self.max_seq_len, self.head_dim,
                                        s_cut.stride()[-2], quantized, reference).view(torch.half)
        assert quantized + self._rest.fill == start_pos + seqlen, \
            f"self.reststartpos + self.restvlen: {quantized + self._rest.fill} != {start_pos + seqlen}"
        o += torch.matmul(s[:, :, :, quantized:start_pos + seqlen],
                          self._rest.data.transpose(1, 2)[:, :, :self._rest.fill, :])
        return o
