"""Ref-counted paged-KV block allocator with a host-side swap pool.

Same role as the reference's BlockManager (engine/block_manager.py:15-117): free-list allocation,
block sharing for prefix hits, append-one-token growth, and an `on_block_freed` hook.  New: blocks
that only the prefix cache still references count as available (an `evictor` callback releases
them on demand), and `swap_space_bytes` is real: `swap_out` / `swap_in` move a sequence's blocks
between the device pool and a pool of host blocks (the reference accepts the option and ignores it,
engine/block_manager.py:29).
"""
from __future__ import annotations

from collections import deque

from .sequence import Sequence


class BlockManager:
    def __init__(self, num_blocks: int, block_size: int, num_cpu_blocks: int = 0):
        assert num_blocks > 0
        self.num_blocks = num_blocks
        self.block_size = block_size
        self.ref_count = [0] * num_blocks
        self.free_block_ids: deque = deque(range(num_blocks))
        self.num_cpu_blocks = num_cpu_blocks
        self.free_cpu_block_ids: deque = deque(range(num_cpu_blocks))
        self.on_block_freed = None          # callable(block_id)
        self.evictor = None                 # callable(n) -> number of blocks released
        self.evictable = None               # callable() -> number of blocks the evictor could release

    # ---- accounting ---------------------------------------------------------
    @property
    def num_free_blocks(self) -> int:
        return len(self.free_block_ids)

    @property
    def num_available_blocks(self) -> int:
        extra = self.evictable() if self.evictable is not None else 0
        return len(self.free_block_ids) + extra

    def _take(self) -> int:
        if not self.free_block_ids and self.evictor is not None:
            self.evictor(1)
        if not self.free_block_ids:
            raise RuntimeError("out of KV blocks")
        b = self.free_block_ids.popleft()
        assert self.ref_count[b] == 0
        self.ref_count[b] = 1
        return b

    def incref(self, block_id: int):
        assert self.ref_count[block_id] > 0
        self.ref_count[block_id] += 1

    def decref(self, block_id: int):
        assert self.ref_count[block_id] > 0, block_id
        self.ref_count[block_id] -= 1
        if self.ref_count[block_id] == 0:
            self.free_block_ids.append(block_id)
            if self.on_block_freed is not None:
                self.on_block_freed(block_id)

    # ---- sequence-level API -----------------------------------------------
    def can_allocate(self, seq: Sequence, num_shared: int = 0) -> bool:
        need = seq.num_blocks - num_shared
        return need <= len(self.free_block_ids) or self.num_available_blocks >= need

    def allocate(self, seq: Sequence):
        assert not seq.block_table
        for _ in range(seq.num_blocks):
            seq.block_table.append(self._take())

    def share_blocks(self, seq: Sequence, blocks: list):
        assert not seq.block_table
        for b in blocks:
            self.incref(b)
            seq.block_table.append(b)

    def allocate_extra(self, seq: Sequence):
        while len(seq.block_table) < seq.num_blocks:
            seq.block_table.append(self._take())

    def can_append(self, seq: Sequence) -> bool:
        need = seq.num_blocks - len(seq.block_table)
        return need <= len(self.free_block_ids) or self.num_available_blocks >= need

    def may_append(self, seq: Sequence):
        self.allocate_extra(seq)

    def deallocate(self, seq: Sequence):
        for b in reversed(seq.block_table):
            self.decref(b)
        seq.block_table = []
        for b in seq.cpu_block_table:
            self.free_cpu_block_ids.append(b)
        seq.cpu_block_table = []

    # ---- swap ---------------------------------------------------------------
    def can_swap_out(self, seq: Sequence) -> bool:
        return len(self.free_cpu_block_ids) >= len(seq.block_table) > 0

    def swap_out(self, seq: Sequence):
        """Move `seq` to host blocks.  Returns (device_blocks, host_blocks) for the copy."""
        dev = list(seq.block_table)
        host = [self.free_cpu_block_ids.popleft() for _ in dev]
        seq.cpu_block_table = host
        for b in reversed(dev):
            self.decref(b)
        seq.block_table = []
        return dev, host

    def can_swap_in(self, seq: Sequence) -> bool:
        # one extra block so the sequence can decode right after coming back
        need = len(seq.cpu_block_table) + 1
        return need <= len(self.free_block_ids) or self.num_available_blocks >= need

    def swap_in(self, seq: Sequence):
        """Bring `seq` back.  Returns (host_blocks, device_blocks) for the copy."""
        host = list(seq.cpu_block_table)
        dev = [self._take() for _ in host]
        seq.block_table = dev
        seq.cpu_block_table = []
        for b in host:
            self.free_cpu_block_ids.append(b)
        return host, dev
