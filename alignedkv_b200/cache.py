"""Decode-time cache orchestration with the surface of the reference's `QuantizedCache_AlignedKV`
(model/KVCache_AlignedKV.py:18-135), free of any `transformers` dependency.

The reference class subclasses `transformers.cache_utils.Cache` of transformers 4.44; that base class changed
incompatibly in later releases, so this stand-in keeps the constructor, attributes and methods the attention
module calls (`auto_compute`, `prefill`, `decoding`, `get_seq_length`, `get_max_length`, `reset`, `.reference`,
`.key_cache`, `.value_cache`) on a plain object.  `config` may be a Hugging Face config or any object with
`num_hidden_layers`, `num_attention_heads`, `num_key_value_heads`, `hidden_size` (or `head_dim`) and
`max_position_embeddings`.
"""
from __future__ import annotations

import math
from typing import Any, Dict, List, Optional, Tuple

import torch
import torch.nn.functional as F

from .extension.k_cache_file import K_Cache_Class
from .extension.v_cache_file import V_Cache_Class

__all__ = ["QuantizedCache_AlignedKV"]


class QuantizedCache_AlignedKV:
    """One AlignedKV plane store per layer; prefill is dense attention, decode runs the aligned kernels."""

    def __init__(self, config, max_batch_size: int, max_cache_len: Optional[int], device, dtype=None) -> None:
        self.max_batch_size = max_batch_size
        self.max_cache_len = config.max_position_embeddings if max_cache_len is None else max_cache_len
        head_dim = getattr(config, "head_dim", None)
        self.head_dim = head_dim if head_dim else config.hidden_size // config.num_attention_heads
        self.dtype = dtype if dtype is not None else torch.float32
        kv_heads = getattr(config, "num_key_value_heads", None)
        self.num_key_value_heads = config.num_attention_heads if kv_heads is None else kv_heads
        assert config.num_attention_heads == self.num_key_value_heads, "We don't support GQA yet."
        self.key_cache: List[K_Cache_Class] = []
        self.value_cache: List[V_Cache_Class] = []
        for idx in range(config.num_hidden_layers):
            self.key_cache.append(K_Cache_Class(max_batch_size, self.max_cache_len, self.num_key_value_heads,
                                                self.head_dim, idx, device, False))
            self.value_cache.append(V_Cache_Class(max_batch_size, self.max_cache_len, self.num_key_value_heads,
                                                  self.head_dim, idx, device, False))
        self.reference = False  # True: every plane is read (the reference's debugging switch)

    def update(self, key_states, value_states, layer_idx: int, cache_kwargs: Optional[Dict[str, Any]] = None
               ) -> Tuple[torch.Tensor, torch.Tensor]:
        raise Exception("This function is not used in AlignedKV")

    def get_seq_length(self, layer_idx: Optional[int] = 0) -> int:
        return self.key_cache[layer_idx].current_cache_len

    def get_max_length(self) -> Optional[int]:
        return self.max_cache_len

    def reset(self):
        for k, v in zip(self.key_cache, self.value_cache):
            k.zerolize()
            v.zerolize()

    # ---- prefill: dense attention; the prompt is written to the planes on the way
    #      (model/KVCache_AlignedKV.py:72-99)
    def prefill_k(self, q, k, seqlen: int, layer_id: int) -> torch.Tensor:
        self.key_cache[layer_id].save(k, 0, seqlen)
        return torch.matmul(q.transpose(1, 2), k.transpose(1, 2).transpose(2, 3)) / math.sqrt(self.head_dim)

    def prefill_v(self, scores, v, seqlen: int, layer_id: int) -> torch.Tensor:
        self.value_cache[layer_id].save(v, 0, seqlen)
        return torch.matmul(scores, v.transpose(1, 2)).transpose(1, 2).contiguous()

    def prefill(self, q, k, v, seqlen: int, mask, layer_id: int) -> torch.Tensor:
        scores = self.prefill_k(q, k, seqlen, layer_id)
        if mask is not None:
            scores = scores + mask
        scores = F.softmax(scores.float(), dim=-1).type_as(q)
        return self.prefill_v(scores, v, seqlen, layer_id)

    # ---- decode: append, aligned q.K^T, fp32 softmax, aligned P.V (model/KVCache_AlignedKV.py:101-124)
    def decoding_k(self, q, k, start_pos: int, seqlen: int, layer_id: int) -> torch.Tensor:
        self.key_cache[layer_id].save(k, start_pos, seqlen)
        return self.key_cache[layer_id].decoding_compute(q, start_pos, seqlen, self.reference)

    def decoding_v(self, scores, v, start_pos: int, seqlen: int, layer_id: int) -> torch.Tensor:
        self.value_cache[layer_id].save(v, start_pos, seqlen)
        return self.value_cache[layer_id].decoding_compute(scores, start_pos, seqlen, self.reference)

    def decoding(self, q, k, v, start_pos: int, seqlen: int, mask, layer_id: int) -> torch.Tensor:
        scores = self.decoding_k(q, k, start_pos, seqlen, layer_id)
        if mask is not None:
            scores[:, :, :, :start_pos + seqlen] += mask
        scores = F.softmax(scores.float(), dim=-1).type_as(q)
        output = self.decoding_v(scores, v, start_pos, seqlen, layer_id)
        return output.view(q.shape[0], q.shape[1], q.shape[2], q.shape[3])

    def auto_compute(self, q, k, v, layer_id: int, mask: Optional[torch.Tensor] = None) -> torch.Tensor:
        seqlen = q.shape[1]
        start_pos = self.get_seq_length(layer_id)
        if mask is not None:
            mask = mask[:, :, :, :start_pos + seqlen]
        if start_pos == 0:
            return self.prefill(q, k, v, seqlen, mask, layer_id)
        return self.decoding(q, k, v, start_pos, seqlen, mask, layer_id)
