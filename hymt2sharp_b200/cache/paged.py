"""Device side of the cache: the pools of key/value blocks of every group of
layers, the block tables that kernels read, and the fixed-size state area.

Storage of one group: [plane, 2 (keys, values), block, kv head, token in block,
head_dim]; a plane is one layer's share.  `tables[g]` is an int32 device matrix
[slot, logical block] → physical block (-1: none).  The host copy of the tables
is the truth; rows that changed are sent before a step runs.

`state` is a byte matrix [slot, state_bytes]: per-sequence state of fixed size
for parts that need it (a recurrent state, a rolling buffer).  A slot's row is
zeroed when the slot is handed out.
"""
from __future__ import annotations

import numpy as np
import torch

from .allocator import CacheBook, CacheError, CacheFull, GroupSpec


class PagedCache:
    def __init__(self, groups: list[GroupSpec], dtype: torch.dtype, device, capacity_tokens: int,
                 block_tokens: int = 64, max_slots: int = 8, state_bytes: int = 0,
                 max_sequence_tokens: int | None = None):
        if capacity_tokens <= 0:
            raise CacheError("capacity_tokens must be positive")
        self.groups = list(groups)
        self.dtype = dtype
        self.device = torch.device(device)
        self.block_tokens = block_tokens
        self.num_blocks = -(-capacity_tokens // block_tokens)
        max_slots = max(1, min(max_slots, self.num_blocks))
        self.book = CacheBook(self.groups, self.num_blocks, block_tokens, max_slots)
        self.storage = [torch.zeros((g.planes, 2, self.num_blocks, g.kv_heads, block_tokens, g.head_dim),
                                    dtype=dtype, device=self.device) for g in self.groups]
        cols = self.num_blocks if max_sequence_tokens is None else -(-max_sequence_tokens // block_tokens)
        self.table_cols = max(1, min(cols, self.num_blocks))
        if max_sequence_tokens is None:
            self.table_cols = min(self.table_cols, 16)  # grows on demand
        self.host_tables = [np.full((max_slots, self.table_cols), -1, dtype=np.int32) for _ in self.groups]
        self.tables = [torch.full((max_slots, self.table_cols), -1, dtype=torch.int32, device=self.device)
                       for _ in self.groups]
        self.state_bytes = int(state_bytes)
        self.state = torch.zeros((max_slots, max(1, self.state_bytes)), dtype=torch.uint8, device=self.device)
        self.layout_version = 0  # bumped when a device tensor that kernels point to is replaced

    # -- sizes ------------------------------------------------------------------
    @property
    def max_slots(self) -> int:
        return self.book.slots.n

    def free_tokens(self) -> int:
        return min(p.free_count for p in self.book.pools) * self.block_tokens if self.groups else 1 << 60

    def bytes_per_token(self) -> int:
        es = torch.empty((), dtype=self.dtype).element_size()
        return sum(2 * g.planes * g.kv_heads * g.head_dim * es for g in self.groups)

    def plane(self, group: int, plane: int) -> tuple[torch.Tensor, torch.Tensor]:
        s = self.storage[group]
        return s[plane, 0], s[plane, 1]

    # -- growth -----------------------------------------------------------------
    def _grow(self, slots: int, cols: int) -> None:
        slots = max(slots, self.max_slots)
        cols = max(cols, self.table_cols)
        if slots == self.max_slots and cols == self.table_cols:
            return
        for g in range(len(self.groups)):
            host = np.full((slots, cols), -1, dtype=np.int32)
            host[: self.host_tables[g].shape[0], : self.table_cols] = self.host_tables[g]
            self.host_tables[g] = host
            self.tables[g] = torch.from_numpy(host).to(self.device)
        if slots > self.state.shape[0]:
            state = torch.zeros((slots, self.state.shape[1]), dtype=torch.uint8, device=self.device)
            state[: self.state.shape[0]] = self.state
            self.state = state
        self.book.slots.grow(slots)
        self.table_cols = cols
        self.layout_version += 1

    # -- slots ------------------------------------------------------------------
    def alloc_slots(self, n: int) -> list[int]:
        if n > self.book.slots.free_count:
            want = self.max_slots - self.book.slots.free_count + n
            if want > self.num_blocks:
                raise CacheFull(f"{want} sequences at once do not fit a cache of {self.num_blocks} blocks")
            self._grow(min(self.num_blocks, max(want, 2 * self.max_slots)), self.table_cols)
        slots = [self.book.alloc_slot() for _ in range(n)]
        if self.state_bytes and slots:
            self.state[torch.tensor(slots, device=self.device)] = 0
        return slots

    def free_slots(self, slots) -> None:
        for s in slots:
            self.book.free_slot(s)
            for g in range(len(self.groups)):
                self.host_tables[g][s, :] = -1
        # the device rows are rewritten when the slot is used again

    def length(self, slot: int) -> int:
        return self.book.length(slot)

    # -- steps ------------------------------------------------------------------
    def begin_step(self, steps: list[tuple[int, int]]) -> None:
        """Blocks for the new tokens of every (slot, new_tokens); all or nothing (CacheFull)."""
        need_cols = max((-(-(self.book.length(s) + n) // self.block_tokens) for s, n in steps), default=0)
        if need_cols > self.num_blocks:
            raise CacheFull(f"a sequence of {need_cols * self.block_tokens} tokens does not fit a cache of "
                            f"{self.num_blocks} blocks of {self.block_tokens}")
        changed = self.book.reserve(steps)
        if need_cols > self.table_cols:
            self._grow(self.max_slots, min(self.num_blocks, max(need_cols, 2 * self.table_cols)))
        for slot, entries in changed.items():
            self._apply(slot, entries)

    def end_step(self, steps: list[tuple[int, int]]) -> None:
        for slot, n in steps:
            entries = self.book.commit(slot, n)
            if entries:
                self._apply(slot, entries)

    def truncate(self, slot: int, length: int) -> None:
        entries = self.book.truncate(slot, length)
        if entries:
            self._apply(slot, entries)

    def _apply(self, slot: int, entries) -> None:
        by_group: dict[int, list[int]] = {}
        for g, logical, phys in entries:
            self.host_tables[g][slot, logical] = phys
            by_group.setdefault(g, []).append(logical)
        # entries past a sequence's length are never read, so a reused slot needs no clearing
        for g, cols in by_group.items():
            self._send_row(slot, [g], min(cols), max(cols) + 1)

    def _send_row(self, slot: int, groups, lo: int, hi: int) -> None:
        for g in groups:
            # through pinned memory and without waiting: a copy from pageable memory makes the host wait for all the work
            # that the stream still holds (steps that were launched ahead).  The pinned piece is a copy of the row as it
            # is now (the host row may change right after) and goes back to torch's pool once the transfer has run.
            src = torch.from_numpy(self.host_tables[g][slot, lo:hi].copy())
            if self.device.type == "cuda":
                src = src.pin_memory()
            self.tables[g][slot, lo:hi].copy_(src, non_blocking=True)
