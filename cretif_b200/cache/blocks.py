"""Bookkeeping of cache storage: a pool of fixed-size token blocks and a set of slots.

Both are plain host-side allocators with strict checks: nothing can be handed
out twice, given back twice, or lost.  The reference has one sequence and one
length counter (src/kv_cache.cu:201-212) and "frees" by resetting that counter
(:237-243); with many sequences the storage has to be accounted for explicitly.
"""
from __future__ import annotations

from typing import List


class CacheError(RuntimeError):
    """Misuse of the cache (unknown slot, double free) or no room left."""


class CacheFull(CacheError):
    """Not enough free blocks or slots for the request; nothing was changed."""


class BlockPool:
    """``n_blocks`` interchangeable blocks, handed out lowest-numbered first."""

    def __init__(self, n_blocks: int):
        if n_blocks <= 0:
            raise ValueError("a block pool needs at least one block")
        self.n_blocks = n_blocks
        self._free: List[int] = list(range(n_blocks - 1, -1, -1))  # pop() gives the lowest
        self._held = [False] * n_blocks

    @property
    def free_count(self) -> int:
        return len(self._free)

    @property
    def held_count(self) -> int:
        return self.n_blocks - len(self._free)

    def take(self, n: int) -> List[int]:
        if n < 0:
            raise ValueError("cannot take a negative number of blocks")
        if n > len(self._free):
            raise CacheFull(f"need {n} cache blocks, only {len(self._free)} of "
                            f"{self.n_blocks} are free")
        out = [self._free.pop() for _ in range(n)]
        for b in out:
            self._held[b] = True
        return out

    def give_back(self, blocks) -> None:
        blocks = list(blocks)
        for b in blocks:
            if not 0 <= b < self.n_blocks:
                raise CacheError(f"block {b} does not belong to this pool")
            if not self._held[b]:
                raise CacheError(f"block {b} is given back but is not held")
        if len(set(blocks)) != len(blocks):
            raise CacheError("a block is given back twice in one call")
        for b in blocks:
            self._held[b] = False
        self._free.extend(sorted(blocks, reverse=True))
        self._free.sort(reverse=True)

    def check(self) -> None:
        """Invariant: every block is either free or held, never both or neither."""
        free = set(self._free)
        if len(free) != len(self._free):
            raise CacheError("a block is on the free list twice")
        for b in range(self.n_blocks):
            if self._held[b] == (b in free):
                raise CacheError(f"block {b} is {'both held and free' if b in free else 'lost'}")


class SlotSet:
    """``n_slots`` sequence handles, lowest-numbered first."""

    def __init__(self, n_slots: int):
        if n_slots <= 0:
            raise ValueError("need at least one slot")
        self.n_slots = n_slots
        self._free: List[int] = list(range(n_slots - 1, -1, -1))
        self._live = [False] * n_slots

    @property
    def free_count(self) -> int:
        return len(self._free)

    def live(self) -> List[int]:
        return [s for s in range(self.n_slots) if self._live[s]]

    def is_live(self, slot: int) -> bool:
        return 0 <= slot < self.n_slots and self._live[slot]

    def take(self) -> int:
        if not self._free:
            raise CacheFull(f"all {self.n_slots} sequence slots are in use")
        s = self._free.pop()
        self._live[s] = True
        return s

    def give_back(self, slot: int) -> None:
        if not 0 <= slot < self.n_slots:
            raise CacheError(f"slot {slot} does not exist (there are {self.n_slots})")
        if not self._live[slot]:
            raise CacheError(f"slot {slot} is freed but is not in use")
        self._live[slot] = False
        self._free.append(slot)
        self._free.sort(reverse=True)

    def check(self) -> None:
        free = set(self._free)
        if len(free) != len(self._free):
            raise CacheError("a slot is on the free list twice")
        for s in range(self.n_slots):
            if self._live[s] == (s in free):
                raise CacheError(f"slot {s} is {'both live and free' if s in free else 'lost'}")
