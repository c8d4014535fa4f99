"""A stand-in for the extension's `cuda_module` that runs the CPU oracle on torch CPU tensors.

Used only by tests: it lets the host-side logic of the cache classes (residual buffering, exponent bookkeeping,
probe inputs, threshold arithmetic) run without a GPU, both for this repository's mirror classes and for the
reference's own Python wrappers when golden vectors are generated."""
import numpy as np
import torch

from oracle import akv_oracle as orc


def _np(t: torch.Tensor) -> np.ndarray:
    assert t.dtype == torch.uint8, f"expected uint8, got {t.dtype}"
    return t.detach().contiguous().numpy()


class OracleCudaModule:
    def __init__(self):
        self.calls = []

    def k_cache_save(self, f8, m4, l4, k_new, bsz, n_kv_heads, n_blocks, n_max_blocks, d_head, d_block, start_pos,
                     seqlen):
        self.calls.append("k_cache_save")
        assert f8.is_contiguous() and m4.is_contiguous() and l4.is_contiguous()
        orc.k_cache_save(f8.numpy(), m4.numpy(), l4.numpy(), _np(k_new), bsz, n_kv_heads, n_blocks, n_max_blocks,
                         d_head, d_block, start_pos, seqlen)

    def k_cache_compute(self, f8, m4, l4, kq, kqmax, q, bsz, n_kv_heads, n_blocks, n_max_blocks, d_head, d_block,
                        seqlen, sqrt_dim, reference):
        self.calls.append("k_cache_compute")
        s, codes = orc.k_cache_compute(_np(f8), _np(m4), _np(l4), _np(kq), _np(kqmax), _np(q), bsz, n_kv_heads,
                                       n_blocks, n_max_blocks, d_head, d_block, seqlen, sqrt_dim, reference)
        self.last_k_codes = codes
        return torch.from_numpy(s.copy())

    def v_cache_save(self, f8, m4, l4, v_new, bsz, n_local_kv_heads, max_seq_len, head_dim, start_pos, seq_len):
        self.calls.append("v_cache_save")
        orc.v_cache_save(f8.numpy(), m4.numpy(), l4.numpy(), _np(v_new), bsz, n_local_kv_heads, max_seq_len, head_dim,
                         start_pos, seq_len)

    def v_cache_test_compute(self, f8, m4, l4, sval, sidx, bsz, n_local_kv_heads, max_seq_len, head_dim, top_max_k):
        self.calls.append("v_cache_test_compute")
        idx = _np(sidx).view(np.int32).reshape(-1, top_max_k).astype(np.int64)
        rows = idx * top_max_k + np.arange(top_max_k)
        if rows.max() >= max_seq_len:   # the reference kernel reads out of bounds here; the result is never used
            return torch.zeros((bsz, n_local_kv_heads, 1, head_dim * 2), dtype=torch.uint8)
        o = orc.v_cache_test_compute(_np(f8), _np(m4), _np(l4), _np(sval), _np(sidx), bsz, n_local_kv_heads,
                                     max_seq_len, head_dim, top_max_k)
        return torch.from_numpy(o.copy())

    def v_cache_compute(self, f8, m4, l4, s, amin, bsz, n_local_kv_heads, max_seq_len, head_dim, s_last_dim, n,
                        reference):
        self.calls.append("v_cache_compute")
        # `s` may be a sliced view: rebuild the rows from its base pointer semantics (row stride s_last_dim halves)
        assert s.dtype == torch.uint8
        rows = torch.zeros((bsz * n_local_kv_heads, max(s_last_dim, 1) * 2), dtype=torch.uint8)
        if n:
            rows[:, :2 * n] = s.reshape(bsz * n_local_kv_heads, -1)[:, :2 * n]
        o, codes = orc.v_cache_compute(_np(f8), _np(m4), _np(l4), rows.numpy(), _np(amin), bsz, n_local_kv_heads,
                                       max_seq_len, head_dim, max(s_last_dim, 1), n, reference)
        self.last_v_codes = codes
        return torch.from_numpy(o.copy())
