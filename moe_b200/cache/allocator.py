"""Host-side bookkeeping of the cache: who holds which slot and which pages.

The bookkeeping itself is C++ (``csrc/host_runtime.cpp``, built with the host
compiler alone, so it is tested on the CPU); the classes here are its Python
face.  A *slot* belongs to one sequence from its first step until it is
released; a *page* holds ``PAGE_TOKENS`` consecutive positions of one sequence
for every layer of one cache group.  Page 0 of every pool is never handed out:
padding rows of a batch point at it.

The reference keeps one flat array of ``ctx`` positions per layer and sequence
(src/model.rs:140-153) and a pool of sessions in its server (src/serve.rs:419-443);
the split into slots and pages is this library's own.
"""
from __future__ import annotations

from ctypes import POINTER, c_char_p, c_int, c_longlong, c_void_p
from typing import List, Sequence, Tuple

import numpy as np

from ..ops import build

PAGE_TOKENS = 64


class CacheError(RuntimeError):
    pass


_lib = None
_IP = POINTER(c_int)


def host_lib():
    """The host runtime library (built on first use)."""
    global _lib
    if _lib is None:
        L = build.load("host")
        P, I, LL = c_void_p, c_int, c_longlong
        sig = {
            "moe_host_page_tokens": ([], I),
            "moe_slotpool_new": ([I], P), "moe_slotpool_delete": ([P], None), "moe_slotpool_acquire": ([P], I),
            "moe_slotpool_release": ([P, I], I), "moe_slotpool_is_held": ([P, I], I), "moe_slotpool_num_free": ([P], I),
            "moe_pagepool_new": ([I], P), "moe_pagepool_delete": ([P], None), "moe_pagepool_alloc": ([P, I, _IP], I),
            "moe_pagepool_free": ([P, _IP, I], I), "moe_pagepool_num_free": ([P], I),
            "moe_ledger_new": ([I, I, _IP, _IP], P), "moe_ledger_delete": ([P], None), "moe_ledger_acquire": ([P], I),
            "moe_ledger_release": ([P, I], I), "moe_ledger_is_held": ([P, I], I), "moe_ledger_length": ([P, I], I),
            "moe_ledger_count": ([P, I, I], I), "moe_ledger_pages": ([P, I, I, _IP, I], I),
            "moe_ledger_extend": ([P, I, I, _IP, I], I), "moe_ledger_truncate": ([P, I, I, _IP], I),
            "moe_ledger_tokens_held": ([P], LL),
            "moe_ledger_reserve": ([P, I, _IP, _IP, _IP, _IP, _IP, I, LL], I),
            "moe_ledger_check": ([P, I, _IP, _IP, _IP, LL], I),
            "moe_pack_step": ([_IP, LL, I, _IP, _IP, _IP, _IP, _IP, _IP, _IP, _IP], LL),
            "moe_pack_decode": ([_IP, I, I, _IP, _IP, _IP, I, I, _IP, _IP, I], I),
            "moe_pack_padded": ([_IP, I, I, I, I, _IP, _IP, _IP, _IP, _IP, _IP, I, I, _IP, I, _IP, I], I),
        }
        for name, (args, res) in sig.items():
            fn = getattr(L, name)
            fn.argtypes, fn.restype = args, res
        L.moe_host_error.argtypes, L.moe_host_error.restype = [], c_char_p
        if L.moe_host_page_tokens() != PAGE_TOKENS:
            raise RuntimeError("the host runtime was built for another page size")
        _lib = L
    return _lib


def _raise(code: int):
    msg = host_lib().moe_host_error().decode()
    raise (ValueError if code == -2 else CacheError)(msg)


def _ok(code: int) -> int:
    if code < 0:
        _raise(code)
    return code


def ints(values: Sequence[int]):
    """A C array of ints (and its length) for the host runtime."""
    n = len(values)
    return (c_int * max(n, 1))(*values), n


def pages_for(length: int, ring_pages: int = 0) -> int:
    """Pages a sequence of ``length`` tokens holds; a ring never holds more than its own size."""
    n = (length + PAGE_TOKENS - 1) // PAGE_TOKENS
    return min(n, ring_pages) if ring_pages else n


class _LedgerSlots:
    def __init__(self, led: "CacheLedger"):
        self._led = led
        self.num_slots = led.num_slots

    def is_held(self, slot: int) -> bool:
        return bool(_lib.moe_ledger_is_held(self._led._h, slot))

    @property
    def num_free(self) -> int:
        return _lib.moe_ledger_count(self._led._h, 0, 0)

    @property
    def num_held(self) -> int:
        return _lib.moe_ledger_count(self._led._h, 1, 0)


class _GroupPool:
    def __init__(self, led: "CacheLedger", group: int):
        self._led, self._g = led, group

    @property
    def num_free(self) -> int:
        return _lib.moe_ledger_count(self._led._h, 2, self._g)

    @property
    def num_pages(self) -> int:
        return _lib.moe_ledger_count(self._led._h, 3, self._g)


class _GroupPages:
    def __init__(self, led: "CacheLedger", group: int):
        self._led, self._g = led, group

    def __getitem__(self, slot: int) -> List[int]:
        n = _ok(_lib.moe_ledger_pages(self._led._h, self._g, slot, None, 0))
        out = (c_int * max(n, 1))()
        _ok(_lib.moe_ledger_pages(self._led._h, self._g, slot, out, n))
        return list(out[:n])


class GroupLedger:
    """Pages of one cache group, per slot: a view of the ledger."""

    def __init__(self, led: "CacheLedger", group: int, ring_pages: int):
        self.pool = _GroupPool(led, group)
        self.ring_pages = ring_pages                     # 0: grows with the sequence
        self.pages = _GroupPages(led, group)


class _Lengths:
    def __init__(self, led: "CacheLedger"):
        self._led = led

    def __getitem__(self, slot: int) -> int:
        n = _lib.moe_ledger_length(self._led._h, slot)
        if n < 0:
            raise KeyError(slot)
        return n

    def __contains__(self, slot) -> bool:
        return bool(_lib.moe_ledger_is_held(self._led._h, slot))


class CacheLedger:
    """Slots, lengths and pages of every group: the host's view of the cache."""

    def __init__(self, num_slots: int, group_pages: List[int], group_ring_pages: List[int]):
        gp, n = ints(group_pages)
        gr, _ = ints(group_ring_pages)
        self.num_slots = num_slots
        self._h = host_lib().moe_ledger_new(num_slots, n, gp, gr)
        if not self._h:
            _raise(-1)
        self.slots = _LedgerSlots(self)
        self.groups = [GroupLedger(self, g, r) for g, r in enumerate(group_ring_pages)]
        self.length = _Lengths(self)

    def __del__(self):
        if getattr(self, "_h", None) and _lib is not None:
            _lib.moe_ledger_delete(self._h)
            self._h = None

    def acquire(self) -> int:
        return _ok(_lib.moe_ledger_acquire(self._h))

    def release(self, slot: int) -> None:
        _ok(_lib.moe_ledger_release(self._h, slot))

    def extend(self, slot: int, new_length: int) -> List[Tuple[int, int, int, int]]:
        """Make room for ``new_length`` tokens in ``slot``.

        Returns the page-table entries that changed as (group, slot, index, page).
        Either every group gets its pages or none does."""
        cap = len(self.groups) * (pages_for(max(new_length, 0)) + 1)
        out = (c_int * (4 * max(cap, 1)))()
        n = _ok(_lib.moe_ledger_extend(self._h, slot, new_length, out, cap))
        return [tuple(out[4 * i:4 * i + 4]) for i in range(n)]

    def reserve(self, slots: Sequence[int], counts: Sequence[int], table_caps: Sequence[int],
                max_tokens: int = 0) -> Tuple[List[int], np.ndarray]:
        """Room for a whole step: sequence ``slots[i]`` brings ``counts[i]`` more tokens.  All or
        nothing.  Returns (each sequence's length before the step, the changed page-table entries
        as an int32 array [n, 4] of (group, slot, index, page))."""
        B = len(slots)
        sl, _ = ints(slots)
        ct, _ = ints(counts)
        caps, _ = ints(table_caps)
        cap = len(self.groups) * sum(max(n, 0) // PAGE_TOKENS + 2 for n in counts)
        starts = (c_int * max(B, 1))()
        upd = np.empty((max(cap, 1), 4), dtype=np.int32)
        n = _ok(_lib.moe_ledger_reserve(self._h, B, sl, ct, caps, starts, upd.ctypes.data_as(_IP), cap, max_tokens))
        if n > cap:
            raise CacheError("internal: more page-table updates than a step can make")
        return list(starts[:B]), upd[:n]

    def check(self, slots: Sequence[int], counts: Sequence[int], table_caps: Sequence[int], max_tokens: int = 0) -> None:
        """Raise what ``reserve`` would raise for this step; change nothing."""
        sl, B = ints(slots)
        ct, _ = ints(counts)
        caps, _ = ints(table_caps)
        _ok(_lib.moe_ledger_check(self._h, B, sl, ct, caps, max_tokens))

    def truncate(self, slot: int, new_length: int, windows: Sequence[int] = ()) -> None:
        """Forget everything at or after ``new_length`` (src/model.rs:176-189).  Pages are
        kept; a ring group that has wrapped can only go back while it still holds the keys that the
        token at ``new_length`` looks back on (``windows``: each group's window, 0 for none; without
        it any rewind of a wrapped ring is refused)."""
        w = ints(list(windows))[0] if len(windows) else None
        _ok(_lib.moe_ledger_truncate(self._h, slot, new_length, w))

    def tokens_held(self) -> int:
        """Tokens the live sequences hold, each rounded up to whole pages."""
        return _lib.moe_ledger_tokens_held(self._h)
