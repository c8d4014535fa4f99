"""Decode attention over a cache that is sharded across the GPUs of one node (one process per GPU).

Two ways to shard, neither of which exists in the reference (it is single-device):

* (batch, KV head) sharding - every (batch, KV head) pair is independent in all operators, so each rank simply owns
  a `DecodeLayer` over its slice of the batch and no collective is on the data path (`shard_batch`).
* sequence sharding for long contexts - `SequenceShardedDecoder`: the cached tokens are split into contiguous,
  64-aligned shards, one per rank.  Every rank receives the query, runs the aligned q.K^T / softmax / P.V over its
  own shard and produces, per (batch, query head), the record (m, l, o): maximum score, sum of exponentials and
  locally normalised output.  One all-gather of those records ((D+2) floats per row and rank, over NCCL) followed by
  a log-sum-exp merge kernel gives every rank the full attention output.  New tokens are appended on the last rank.
  Read decisions are taken from each shard's own softmax and magnitude probe, so they can differ from a
  single-device run over the whole sequence; the merged output is compared against fp32 dense attention.
"""
from __future__ import annotations

import torch

from . import _lib

__all__ = ["shard_bounds", "shard_batch", "SequenceShardedDecoder"]

BLOCK = 64


def shard_bounds(n_tokens: int, world: int, block: int = BLOCK):
    """Contiguous token ranges [lo, hi) per rank: whole blocks, as even as possible, the remainder on the last."""
    nblk = n_tokens // block
    per, extra = divmod(nblk, world)
    bounds, lo = [], 0
    for r in range(world):
        hi = lo + (per + (1 if r < extra else 0)) * block
        bounds.append((lo, hi))
        lo = hi
    bounds[-1] = (bounds[-1][0], n_tokens)
    return bounds


def shard_batch(bsz: int, world: int, rank: int):
    """Rows [lo, hi) of the batch owned by `rank` under (batch, KV head) sharding."""
    per, extra = divmod(bsz, world)
    lo = rank * per + min(rank, extra)
    return lo, lo + per + (1 if rank < extra else 0)


class _CudaBackend:
    """Local step and merge through the C ABI."""

    def __init__(self, bsz, max_local_len, n_kv_heads, head_dim, device, n_q_heads, v_mode):
        from .decode import DecodeLayer
        self.layer = DecodeLayer(bsz, max_local_len, n_kv_heads, head_dim, device, n_q_heads=n_q_heads, v_mode=v_mode)
        self.lib = _lib.load()
        self.device = torch.device(device)

    def prefill(self, k, v):
        self.layer.prefill(k, v)

    def record(self, q, k, v, append):
        return self.layer.decode(q, k, v, append=append, packed=True)

    def merge(self, gathered, rows, head_dim):
        out = torch.empty((rows, head_dim), dtype=torch.half, device=self.device)
        with torch.cuda.device(self.device):
            rc = self.lib.akv_lse_merge(gathered.data_ptr(), out.data_ptr(), gathered.shape[0], rows, head_dim,
                                        torch.cuda.current_stream(self.device).cuda_stream)
        _lib.check("lse_merge", rc)
        return out


class SequenceShardedDecoder:
    """One layer's cache with the sequence split across the ranks of `group` (see the module docstring).

    backend: object with prefill(k, v), record(q, k, v, append) -> fp32 [B*Hq, D+2] and merge(gathered, rows, D);
    the default drives the CUDA kernels.  Tests substitute a CPU implementation to exercise the protocol with gloo."""

    def __init__(self, bsz: int, prompt_len: int, max_new_tokens: int, n_kv_heads: int, head_dim: int, device,
                 n_q_heads: int | None = None, v_mode: str = "order_free", group=None, backend=None):
        import torch.distributed as dist
        self.dist = dist
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.B, self.D = bsz, head_dim
        self.Hq = n_kv_heads if n_q_heads is None else n_q_heads
        self.bounds = shard_bounds(prompt_len, self.world)
        lo, hi = self.bounds[self.rank]
        self.is_last = self.rank == self.world - 1
        self.local_len = hi - lo
        max_local = self.local_len + (max_new_tokens if self.is_last else 0)
        max_local = max(BLOCK, -(-max_local // BLOCK) * BLOCK)
        self.backend = backend if backend is not None else _CudaBackend(bsz, max_local, n_kv_heads, head_dim, device,
                                                                        self.Hq, v_mode)

    def prefill(self, k_shard, v_shard) -> None:
        """k_shard, v_shard: this rank's tokens [B, hi-lo, H, D] of the prompt (ranks load their own shard)."""
        if k_shard.shape[1] != self.local_len:
            raise ValueError(f"rank {self.rank} owns {self.local_len} tokens, got {k_shard.shape[1]}")
        if self.local_len:
            self.backend.prefill(k_shard, v_shard)

    def decode(self, q, k_new, v_new):
        """q [B,1,Hq,D], k_new / v_new [B,1,H,D] (used on the last rank only) -> merged output [B,1,Hq,D] on every
        rank."""
        rec = self.backend.record(q, k_new if self.is_last else None, v_new if self.is_last else None, self.is_last)
        rows = self.B * self.Hq
        if self.world == 1:
            gathered = rec.reshape(1, rows, self.D + 2)
        else:
            flat = torch.empty((self.world * rows, self.D + 2), dtype=rec.dtype, device=rec.device)
            self.dist.all_gather_into_tensor(flat, rec.contiguous(), group=self.group)   # rank-major concatenation
            gathered = flat.view(self.world, rows, self.D + 2)
        return self.backend.merge(gathered, rows, self.D).reshape(self.B, 1, self.Hq, self.D)
