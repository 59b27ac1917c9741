"""Block allocator and block tables for the paged KV cache.

The reference's engine lists a "KV cache" without code (reports/11_custom_engine.md:10-20);
in its shipped path the cache is vLLM's.  Here: fixed-size blocks (16 tokens by default), a
free list on the host, and a device-resident block table [max_batch, max_blocks_per_seq]
that the attention kernel reads.  Block 0 is never handed out: idle batch rows and graph
warm-up point at it, so a stray write can never land in a live sequence.
"""
from __future__ import annotations

from typing import List

import torch


class BlockManager:
    def __init__(self, num_blocks: int, block_size: int, max_batch: int, max_blocks_per_seq: int, device):
        self.num_blocks, self.block_size = num_blocks, block_size
        self.max_batch, self.max_blocks_per_seq = max_batch, max_blocks_per_seq
        self.free: List[int] = list(range(num_blocks - 1, 0, -1))   # block 0 reserved
        self.tables_host = torch.zeros(max_batch, max_blocks_per_seq, dtype=torch.int32).pin_memory() \
            if torch.cuda.is_available() else torch.zeros(max_batch, max_blocks_per_seq, dtype=torch.int32)
        self.tables = torch.zeros(max_batch, max_blocks_per_seq, dtype=torch.int32, device=device)
        self.owned: List[List[int]] = [[] for _ in range(max_batch)]

    def blocks_needed(self, tokens: int) -> int:
        return (tokens + self.block_size - 1) // self.block_size

    def reserve(self, row: int, tokens: int) -> None:
        """Make sure batch row ``row`` owns blocks for ``tokens`` tokens."""
        need = self.blocks_needed(tokens)
        if need > self.max_blocks_per_seq:
            raise ValueError(f"sequence of {tokens} tokens exceeds max_seq_len")
        have = self.owned[row]
        while len(have) < need:
            if not self.free:
                raise RuntimeError("KV cache is out of blocks")
            b = self.free.pop()
            self.tables_host[row, len(have)] = b
            have.append(b)

    def release(self, row: int) -> None:
        self.free.extend(reversed(self.owned[row]))
        self.owned[row] = []
        self.tables_host[row].zero_()

    def release_all(self) -> None:
        for r in range(self.max_batch):
            if self.owned[r]:
                self.release(r)

    def slot(self, row: int, pos: int) -> int:
        return int(self.tables_host[row, pos // self.block_size]) * self.block_size + pos % self.block_size

    def sync_to_device(self) -> None:
        self.tables.copy_(self.tables_host, non_blocking=True)
