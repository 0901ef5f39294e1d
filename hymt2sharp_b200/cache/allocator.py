"""Host-side bookkeeping of the cache: which sequence holds which slot and which
blocks.  Pure Python, no device: it decides, the device tensors follow.

A *slot* is one sequence's place in a batch: its length, and for every group of
layers a list of block numbers (logical block i of the sequence → physical
block of that group's pool, or -1 once a window group has dropped it).  A
*group* is a set of layers with the same needs: "full" keeps every key, "window"
keeps the last `window` positions and gives older blocks back as the sequence
grows.  Slots and blocks are given back when a sequence ends and are used again.
"""
from __future__ import annotations

from dataclasses import dataclass, field


class CacheError(RuntimeError):
    pass


class CacheFull(CacheError):
    """Not enough free blocks or slots; nothing was changed."""


@dataclass(frozen=True)
class GroupSpec:
    """What one group of layers needs from the cache."""
    kind: str               # "full" or "window"
    kv_heads: int
    head_dim: int
    planes: int             # layers (schedule entries) that store keys and values here
    window: int = 0         # for kind "window": positions that stay visible

    def key(self):
        return (self.kind, self.kv_heads, self.head_dim, self.window)


class FreeList:
    """Numbers 0..n-1, each either free or held; lowest number first."""

    def __init__(self, n: int, what: str):
        self.n = n
        self.what = what
        self._free = list(range(n - 1, -1, -1))
        self._held = [False] * n

    def grow(self, n: int) -> None:
        if n > self.n:
            self._free = list(range(n - 1, self.n - 1, -1)) + self._free
            self._held += [False] * (n - self.n)
            self.n = n

    @property
    def free_count(self) -> int:
        return len(self._free)

    def take(self) -> int:
        if not self._free:
            raise CacheFull(f"no free {self.what} left (all {self.n} are held)")
        i = self._free.pop()
        self._held[i] = True
        return i

    def give(self, i: int) -> None:
        if not (0 <= i < self.n):
            raise CacheError(f"{self.what} {i} does not exist")
        if not self._held[i]:
            raise CacheError(f"{self.what} {i} is freed twice")
        self._held[i] = False
        self._free.append(i)

    def is_held(self, i: int) -> bool:
        return self._held[i]


@dataclass
class Sequence:
    slot: int
    length: int = 0
    blocks: list = field(default_factory=list)   # per group: list of physical block numbers


class CacheBook:
    """Slots and blocks of every group."""

    def __init__(self, groups: list[GroupSpec], blocks_per_group: int, block_tokens: int, max_slots: int):
        if block_tokens <= 0 or blocks_per_group <= 0 or max_slots <= 0:
            raise CacheError("block_tokens, blocks_per_group and max_slots must be positive")
        self.groups = list(groups)
        self.block_tokens = block_tokens
        self.blocks_per_group = blocks_per_group
        self.slots = FreeList(max_slots, "slot")
        self.pools = [FreeList(blocks_per_group, f"block of group {i}") for i in range(len(groups))]
        self.sequences: dict[int, Sequence] = {}

    # -- slots ----------------------------------------------------------------
    def alloc_slot(self) -> int:
        slot = self.slots.take()
        self.sequences[slot] = Sequence(slot, 0, [[] for _ in self.groups])
        return slot

    def free_slot(self, slot: int) -> None:
        seq = self._seq(slot)
        for g, blocks in enumerate(seq.blocks):
            for b in blocks:
                if b >= 0:
                    self.pools[g].give(b)
        del self.sequences[slot]
        self.slots.give(slot)

    def _seq(self, slot: int) -> Sequence:
        try:
            return self.sequences[slot]
        except KeyError:
            raise CacheError(f"slot {slot} is not held") from None

    def length(self, slot: int) -> int:
        return self._seq(slot).length

    # -- blocks ---------------------------------------------------------------
    def _first_needed_block(self, group: GroupSpec, length_before: int) -> int:
        """The first logical block that a step starting at `length_before` can still read."""
        if group.kind != "window":
            return 0
        first_key = max(0, length_before - group.window + 1)
        return first_key // self.block_tokens

    def blocks_needed(self, slot: int, new_tokens: int) -> list[int]:
        seq = self._seq(slot)
        total = -(-(seq.length + new_tokens) // self.block_tokens)
        return [max(0, total - len(blocks)) for blocks in seq.blocks]

    def reserve(self, steps: list[tuple[int, int]]) -> dict[int, list[tuple[int, int, int]]]:
        """Blocks for the new tokens of a whole step, all or nothing.
        `steps` = [(slot, new_tokens)].  Returns, per slot, the table entries that changed:
        (group, logical block, physical block)."""
        need = [0] * len(self.groups)
        seen = set()
        for slot, n in steps:
            if slot in seen:
                raise CacheError(f"slot {slot} appears twice in one step")
            seen.add(slot)
            if n < 0:
                raise CacheError("a step cannot take tokens away")
            for g, k in enumerate(self.blocks_needed(slot, n)):
                need[g] += k
        for g, k in enumerate(need):
            if k > self.pools[g].free_count:
                raise CacheFull(f"the step needs {k} more blocks of {self.block_tokens} tokens in group {g}, "
                                f"{self.pools[g].free_count} of {self.pools[g].n} are free")
        changed: dict[int, list[tuple[int, int, int]]] = {}
        for slot, n in steps:
            seq = self.sequences[slot]
            for g, k in enumerate(self.blocks_needed(slot, n)):
                for _ in range(k):
                    b = self.pools[g].take()
                    seq.blocks[g].append(b)
                    changed.setdefault(slot, []).append((g, len(seq.blocks[g]) - 1, b))
        return changed

    def commit(self, slot: int, new_tokens: int) -> list[tuple[int, int, int]]:
        """The step ran: the sequence is `new_tokens` longer.  Window groups give back the
        blocks that no later step can read.  Returns changed table entries (physical -1)."""
        seq = self._seq(slot)
        seq.length += new_tokens
        for blocks in seq.blocks:
            if seq.length > len(blocks) * self.block_tokens:
                seq.length -= new_tokens
                raise CacheError(f"slot {slot}: {new_tokens} tokens were committed but not reserved")
        changed = []
        for g, group in enumerate(self.groups):
            first = self._first_needed_block(group, seq.length)
            for i in range(min(first, len(seq.blocks[g]))):
                b = seq.blocks[g][i]
                if b >= 0:
                    self.pools[g].give(b)
                    seq.blocks[g][i] = -1
                    changed.append((g, i, -1))
        return changed

    def truncate(self, slot: int, length: int) -> list[tuple[int, int, int]]:
        """Forget everything from position `length` on (src/HyMT2Sharp/HunyuanDenseModel.cs:187-240)."""
        seq = self._seq(slot)
        if not (0 <= length <= seq.length):
            raise CacheError(f"slot {slot}: cannot truncate {seq.length} tokens to {length}")
        keep = -(-length // self.block_tokens)
        changed = []
        for g, group in enumerate(self.groups):
            first = self._first_needed_block(group, length)
            if any(b < 0 for b in seq.blocks[g][first:keep]):
                raise CacheError(f"slot {slot}: group {g} has already dropped blocks that a truncation to {length} needs")
            while len(seq.blocks[g]) > keep:
                b = seq.blocks[g].pop()
                if b >= 0:
                    self.pools[g].give(b)
                changed.append((g, len(seq.blocks[g]), -1))
        seq.length = length
        return changed

    # -- checks (used by tests) -----------------------------------------------
    def audit(self) -> None:
        """Every block is free or held by exactly one sequence; every held slot has a sequence."""
        for g, pool in enumerate(self.pools):
            held = [b for s in self.sequences.values() for b in s.blocks[g] if b >= 0]
            if len(held) != len(set(held)):
                raise CacheError(f"group {g}: a block is held twice")
            if len(held) + pool.free_count != pool.n:
                raise CacheError(f"group {g}: {pool.n - len(held) - pool.free_count} blocks are lost")
            for b in held:
                if not pool.is_held(b):
                    raise CacheError(f"group {g}: block {b} is in use but marked free")
        if len(self.sequences) + self.slots.free_count != self.slots.n:
            raise CacheError("a slot is lost")
