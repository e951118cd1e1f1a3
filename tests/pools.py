"""The slot and page pools of the host runtime on their own (the ledger holds one of each kind
inside the C++ library; the product reaches them only through the ledger).  These thin classes let
the tests drive the pools' C entry points directly."""
from ctypes import c_int
from typing import List

from moe_b200.cache import allocator
from moe_b200.cache.allocator import _ok, _raise, host_lib, ints


def _lib():
    return host_lib()


class SlotPool:
    """Slots 0 .. n-1; each is free or held by exactly one sequence."""

    def __init__(self, num_slots: int):
        self.num_slots = num_slots
        self._h = _lib().moe_slotpool_new(num_slots)
        if not self._h:
            _raise(-1)

    def __del__(self):
        if getattr(self, "_h", None) and allocator._lib is not None:
            _lib().moe_slotpool_delete(self._h)
            self._h = None

    def acquire(self) -> int:
        return _ok(_lib().moe_slotpool_acquire(self._h))

    def release(self, slot: int) -> None:
        _ok(_lib().moe_slotpool_release(self._h, slot))

    def is_held(self, slot: int) -> bool:
        return bool(_lib().moe_slotpool_is_held(self._h, slot))

    @property
    def num_free(self) -> int:
        return _lib().moe_slotpool_num_free(self._h)

    @property
    def num_held(self) -> int:
        return self.num_slots - self.num_free


class PagePool:
    """Pages 1 .. n-1 of one cache group (page 0 is the scratch page)."""

    def __init__(self, num_pages: int):
        self.num_pages = num_pages
        self._h = _lib().moe_pagepool_new(num_pages)
        if not self._h:
            _raise(-1)

    def __del__(self):
        if getattr(self, "_h", None) and allocator._lib is not None:
            _lib().moe_pagepool_delete(self._h)
            self._h = None

    def alloc(self, n: int) -> List[int]:
        out = (c_int * max(n, 1))()
        got = _ok(_lib().moe_pagepool_alloc(self._h, n, out))
        return list(out[:got])

    def free(self, pages: List[int]) -> None:
        arr, n = ints(pages)
        _ok(_lib().moe_pagepool_free(self._h, arr, n))

    @property
    def num_free(self) -> int:
        return _lib().moe_pagepool_num_free(self._h)


