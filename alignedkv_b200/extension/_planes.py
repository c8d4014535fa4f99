"""Pieces shared by the K and V plane stores: constants, exponent extraction, residual-token buffering."""
from __future__ import annotations

import torch

# One K channel row of a block holds 256 bits of high bytes = 64 tokens (extension/k_cache_file.py:5-6).
bits_in_a_channel = 256
column_block = bits_in_a_channel // 4


def cdiv(a: int, b: int) -> int:
    return -(-a // b)


def exponent_field(x: torch.Tensor) -> torch.Tensor:
    """5-bit biased exponent of every fp16 element, as uint8 (the reference's
    `(x.view(int16) >> 10).to(uint8) & 0x1F`, e.g. extension/k_cache_file.py:77-78,98-99,136)."""
    return (x.view(torch.int16) >> 10).to(torch.uint8) & 0x1F


class ResidualBuffer:
    """The fp16 staging area for tokens that do not yet fill a 64-token block.

    The reference keeps them in `restk` / `restv` of shape [bsz, 64, heads, head_dim] with a fill count and the
    position of the first buffered token (extension/k_cache_file.py:92-96,100-118; extension/v_cache_file.py:92-96,
    101-116).  Only whole blocks ever reach the plane writers.
    """

    def __init__(self, bsz: int, heads: int, head_dim: int, device):
        self.shape = (bsz, column_block, heads, head_dim)
        self.device = device
        self.data: torch.Tensor | None = None
        self.fill = 0
        self.start = 0

    def fresh(self) -> torch.Tensor:
        self.data = torch.zeros(self.shape, dtype=torch.half, device=self.device)
        return self.data

    def load_tail(self, new: torch.Tensor, seqlen: int) -> None:
        """After a prefill: keep the seqlen % 64 trailing tokens."""
        tail = seqlen % column_block
        self.fresh()
        self.data[:, :tail, :, :] = new[:, seqlen - tail:, :]
        self.fill = tail
        self.start = seqlen - tail

    def push(self, new: torch.Tensor, seqlen: int) -> bool:
        """Append decode tokens; True when the buffer now holds a whole block."""
        self.data[:, self.fill:self.fill + seqlen, :, :] = new
        self.fill += seqlen
        return self.fill == column_block

    def advance(self) -> None:
        """The buffered block has been written to the planes."""
        self.fill = 0
        self.start += column_block
        self.fresh()
