"""Page allocator for the paged KV cache.

Same observable behaviour as ``engines/nano_dvlm/nanovllm/engine/block_manager.py``
with prefix-cache hashing off, which is how the reference runs (its hash line
is commented out at ``block_manager.py:65-66`` so every allocation misses):
pages are handed out from the front of a FIFO free list and returned to its
back in reverse table order.
"""
from __future__ import annotations

from collections import deque

from .sequence import Sequence


class BlockManager:

    def __init__(self, num_blocks: int, block_size: int):
        self.block_size = block_size
        self.num_blocks = num_blocks
        self.free_block_ids: deque[int] = deque(range(num_blocks))
        self.used_block_ids: set[int] = set()

    def _take(self) -> int:
        block_id = self.free_block_ids.popleft()
        self.used_block_ids.add(block_id)
        return block_id

    def can_allocate(self, seq: Sequence) -> bool:
        return len(self.free_block_ids) >= seq.num_blocks

    def allocate(self, seq: Sequence):
        if seq.block_table:
            raise AssertionError("sequence already holds pages")
        for _ in range(seq.num_blocks):
            seq.block_table.append(self._take())

    def deallocate(self, seq: Sequence):
        for block_id in reversed(seq.block_table):
            self.used_block_ids.remove(block_id)
            self.free_block_ids.append(block_id)
        seq.num_cached_tokens = 0
        seq.block_table.clear()

    def can_append(self, seq: Sequence) -> bool:
        return len(self.free_block_ids) >= int(seq.need_new_block())

    def may_append(self, seq: Sequence):
        if seq.need_new_block():
            seq.block_table.append(self._take())
