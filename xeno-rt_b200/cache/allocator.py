"""Host-side allocators of the cache: blocks of token positions, and slots (one a sequence).

Both are plain free lists with the bookkeeping that makes misuse an error instead of a silent
fault: nothing is handed out twice, nothing is taken back twice, and what is free plus what is
held is always everything.
"""
from __future__ import annotations

from ..core import CacheError


class BlockAllocator:
    """``count`` blocks, numbered from 0.  Lowest numbers are handed out first, and a block that
    was given back is used again before a block that never was, so reuse shows early in tests."""

    def __init__(self, count: int):
        if count < 0:
            raise CacheError(f"block count {count} is negative")
        self.count = count
        self._free = list(range(count - 1, -1, -1))  # a stack; pop() gives the lowest first
        self._held = [False] * count

    @property
    def free(self) -> int:
        return len(self._free)

    @property
    def held(self) -> int:
        return self.count - len(self._free)

    def take(self, n: int) -> list[int]:
        if n < 0:
            raise CacheError(f"cannot take {n} blocks")
        if n > len(self._free):
            raise CacheError(f"the cache is full: {n} blocks are needed, {len(self._free)} of {self.count} are free")
        out = [self._free.pop() for _ in range(n)]
        for b in out:
            self._held[b] = True
        return out

    def give_back(self, blocks) -> None:
        blocks = list(blocks)
        for b in blocks:
            if not (0 <= b < self.count):
                raise CacheError(f"block {b} does not exist")
            if not self._held[b]:
                raise CacheError(f"block {b} is given back twice")
            self._held[b] = False
        # sorted so that the lowest comes out first again
        self._free.extend(sorted(blocks, reverse=True))

    def check(self) -> None:
        """Raises if the books do not balance (used by tests)."""
        if sorted(self._free) != [b for b in range(self.count) if not self._held[b]]:
            raise CacheError("block allocator: the free list and the held marks disagree")


class SlotAllocator:
    """``count`` slots; a slot is the handle of one live sequence."""

    def __init__(self, count: int):
        self._blocks = BlockAllocator(count)

    @property
    def count(self) -> int:
        return self._blocks.count

    @property
    def free(self) -> int:
        return self._blocks.free

    def open(self) -> int:
        if self._blocks.free == 0:
            raise CacheError(f"no free slot: all {self.count} slots hold live sequences")
        return self._blocks.take(1)[0]

    def close(self, slot: int) -> None:
        try:
            self._blocks.give_back([slot])
        except CacheError:
            raise CacheError(f"slot {slot} is not open (closed twice, or never opened)") from None

    def is_open(self, slot: int) -> bool:
        return 0 <= slot < self.count and self._blocks._held[slot]

    def check(self) -> None:
        self._blocks.check()
