"""Host-side bookkeeping of the cache: who holds which slot and which pages.

Nothing here touches the device, so it is tested on the CPU.  A *slot* belongs
to one sequence from its first step until it is released; a *page* holds
``PAGE_TOKENS`` consecutive positions of one sequence for every layer of one
cache group.  Page 0 of every pool is never handed out: padding rows of a batch
point at it.

The reference keeps one flat array of ``ctx`` positions per layer and sequence
(src/model.rs:140-153) and a pool of sessions in its server (src/serve.rs:419-443);
the split into slots and pages is this library's own.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

PAGE_TOKENS = 64


class CacheError(RuntimeError):
    pass


class SlotPool:
    """Slots 0 .. n-1; each is free or held by exactly one sequence."""

    def __init__(self, num_slots: int):
        if num_slots <= 0:
            raise CacheError("a cache needs at least one slot")
        self.num_slots = num_slots
        self._free: List[int] = list(range(num_slots - 1, -1, -1))   # pop() hands out the lowest first
        self._held = [False] * num_slots

    def acquire(self) -> int:
        if not self._free:
            raise CacheError(f"all {self.num_slots} slots are in use")
        s = self._free.pop()
        self._held[s] = True
        return s

    def release(self, slot: int) -> None:
        if not 0 <= slot < self.num_slots:
            raise CacheError(f"slot {slot} does not exist")
        if not self._held[slot]:
            raise CacheError(f"slot {slot} is not held (released twice?)")
        self._held[slot] = False
        self._free.append(slot)

    def is_held(self, slot: int) -> bool:
        return 0 <= slot < self.num_slots and self._held[slot]

    @property
    def num_free(self) -> int:
        return len(self._free)

    @property
    def num_held(self) -> int:
        return self.num_slots - len(self._free)


class PagePool:
    """Pages 1 .. n-1 of one cache group (page 0 is the scratch page)."""

    def __init__(self, num_pages: int):
        if num_pages < 2:
            raise CacheError("a page pool needs the scratch page and at least one more")
        self.num_pages = num_pages
        self._free: List[int] = list(range(num_pages - 1, 0, -1))
        self._held = [False] * num_pages

    def alloc(self, n: int) -> List[int]:
        if n > len(self._free):
            raise CacheError(
                f"the cache is full: {n} more pages of {PAGE_TOKENS} tokens wanted, {len(self._free)} free "
                f"of {self.num_pages - 1}"
            )
        out = [self._free.pop() for _ in range(n)]
        for p in out:
            self._held[p] = True
        return out

    def free(self, pages: List[int]) -> None:
        for p in pages:
            if not 0 < p < self.num_pages:
                raise CacheError(f"page {p} does not exist")
            if not self._held[p]:
                raise CacheError(f"page {p} is not held (freed twice?)")
        for p in pages:
            self._held[p] = False
            self._free.append(p)

    @property
    def num_free(self) -> int:
        return len(self._free)


def pages_for(length: int, ring_pages: int = 0) -> int:
    """Pages a sequence of ``length`` tokens holds; a ring never holds more than its own size."""
    n = (length + PAGE_TOKENS - 1) // PAGE_TOKENS
    return min(n, ring_pages) if ring_pages else n


@dataclass
class GroupLedger:
    """Pages of one cache group, per slot."""

    pool: PagePool
    ring_pages: int                      # 0: grows with the sequence
    pages: Dict[int, List[int]] = field(default_factory=dict)


class CacheLedger:
    """Slots, lengths and pages of every group: the host's view of the cache."""

    def __init__(self, num_slots: int, group_pages: List[int], group_ring_pages: List[int]):
        self.slots = SlotPool(num_slots)
        self.groups = [GroupLedger(PagePool(n), r) for n, r in zip(group_pages, group_ring_pages)]
        self.length: Dict[int, int] = {}

    def acquire(self) -> int:
        s = self.slots.acquire()
        self.length[s] = 0
        for g in self.groups:
            g.pages[s] = []
        return s

    def release(self, slot: int) -> None:
        if not self.slots.is_held(slot):
            raise CacheError(f"slot {slot} is not held (released twice?)")
        for g in self.groups:
            g.pool.free(g.pages.pop(slot))
        del self.length[slot]
        self.slots.release(slot)

    def extend(self, slot: int, new_length: int) -> List[Tuple[int, int, int, int]]:
        """Make room for ``new_length`` tokens in ``slot``.

        Returns the page-table entries that changed as (group, slot, index, page).
        Either every group gets its pages or none does."""
        if not self.slots.is_held(slot):
            raise CacheError(f"slot {slot} is not held")
        if new_length < self.length[slot]:
            raise CacheError("extend cannot shrink a sequence; use truncate")
        wants = []
        for g in self.groups:
            need = pages_for(new_length, g.ring_pages) - len(g.pages[slot])
            if need > g.pool.num_free:
                raise CacheError(
                    f"the cache is full: slot {slot} needs {need} more pages of {PAGE_TOKENS} tokens, "
                    f"{g.pool.num_free} free"
                )
            wants.append(max(need, 0))
        updates = []
        for gi, (g, need) in enumerate(zip(self.groups, wants)):
            if need:
                base = len(g.pages[slot])
                new = g.pool.alloc(need)
                g.pages[slot].extend(new)
                updates.extend((gi, slot, base + i, p) for i, p in enumerate(new))
        self.length[slot] = new_length
        return updates

    def truncate(self, slot: int, new_length: int) -> None:
        """Forget everything at or after ``new_length`` (src/model.rs:176-189).  Pages are
        kept; a ring group can only go back while the kept prefix is still inside it."""
        if not self.slots.is_held(slot):
            raise CacheError(f"slot {slot} is not held")
        cur = self.length[slot]
        if new_length > cur:
            raise CacheError("truncate cannot lengthen a sequence")
        for g in self.groups:
            if g.ring_pages and new_length < cur and cur > g.ring_pages * PAGE_TOKENS:
                raise CacheError("a windowed cache that has wrapped cannot be rewound")
        self.length[slot] = new_length

    def tokens_held(self) -> int:
        """Tokens the live sequences hold, each rounded up to whole pages."""
        return sum(pages_for(n) * PAGE_TOKENS for n in self.length.values())
