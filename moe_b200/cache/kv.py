"""Device storage of the cache: keys and values in pages, and per-sequence state.

Layers whose mixers ask for the same record (kv heads, head size, window) form a
*group* with storage and a page table of its own.  A group without a window
keeps every position; a windowed group is a ring of ``ceil(window / 64)`` pages
per sequence, position p living at ``p mod ring``.

One layer of a group is laid out ``[page][kv_head][64][head_dim]`` for keys and
the same for values, so that the 64 positions of a page are contiguous per head.

Beside the pages, every cache entry may own *state of fixed size* per sequence
(``[slots + 1, *shape]``), which is where a recurrent mixer would keep its
carry and where the sampler keeps its random-number state.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import torch

from .allocator import PAGE_TOKENS, CacheError, CacheLedger


@dataclass(frozen=True)
class KVRequest:
    """What a mixer needs stored per position."""

    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class StateRequest:
    """State of fixed size per sequence."""

    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


class CacheGroup:
    def __init__(self, index: int, req: KVRequest, cache_ids: List[int], num_pages: int, max_slots: int,
                 max_pages_per_seq: int, dtype: torch.dtype, device):
        self.index = index
        self.num_kv_heads, self.head_dim, self.window = req.num_kv_heads, req.head_dim, req.window
        self.cache_ids = list(cache_ids)
        self.page_size = PAGE_TOKENS
        self.ring_pages = 0 if req.window is None else -(-req.window // PAGE_TOKENS)
        self.ring = self.ring_pages * PAGE_TOKENS
        self.num_pages = num_pages
        self.dtype = dtype
        self.max_pages_per_seq = max_pages_per_seq
        # [layer][k|v][page][kv_head][pos][dim]
        self.storage = torch.zeros(
            (len(cache_ids), 2, num_pages, req.num_kv_heads, PAGE_TOKENS, req.head_dim), dtype=dtype, device=device
        )
        # one row per slot plus the padding row, whose entries stay 0 (the scratch page)
        self.table = torch.zeros((max_slots + 1, max_pages_per_seq), dtype=torch.int32, device=device)

    def bytes(self) -> int:
        return self.storage.numel() * self.storage.element_size()


class CacheView:
    """One layer's keys and values inside its group."""

    def __init__(self, group: CacheGroup, layer: int):
        self.group = group
        self.layer = layer
        self.k = group.storage[layer, 0]
        self.v = group.storage[layer, 1]


class KVCache:
    """Slots, pages and fixed-size state for one model on one device.

    ``max_tokens`` is the most tokens that live sequences may hold at any time,
    each sequence's count rounded up to a multiple of 64."""

    def __init__(self, kv_requests: Dict[int, Optional[KVRequest]], state_requests: Dict[int, Optional[StateRequest]],
                 max_tokens: int, max_slots: int, dtype: torch.dtype, device):
        if max_tokens <= 0:
            raise CacheError("max_tokens must be positive")
        self.device = device
        self.dtype = dtype
        self.max_slots = max_slots
        self.max_tokens = -(-max_tokens // PAGE_TOKENS) * PAGE_TOKENS
        budget_pages = self.max_tokens // PAGE_TOKENS
        by_key: Dict[KVRequest, List[int]] = {}
        for cid, req in kv_requests.items():
            if req is not None:
                by_key.setdefault(req, []).append(cid)
        self.groups: List[CacheGroup] = []
        self._views: Dict[int, CacheView] = {}
        for gi, (req, cids) in enumerate(by_key.items()):
            ring_pages = 0 if req.window is None else -(-req.window // PAGE_TOKENS)
            if ring_pages:
                per_seq = min(ring_pages, budget_pages)
                pages = min(budget_pages, max_slots * ring_pages) + 1
            else:
                per_seq = budget_pages
                pages = budget_pages + 1
            g = CacheGroup(gi, req, cids, pages, max_slots, per_seq, dtype, device)
            self.groups.append(g)
            for li, cid in enumerate(cids):
                self._views[cid] = CacheView(g, li)
        self.ledger = CacheLedger(max_slots, [g.num_pages for g in self.groups], [g.ring_pages for g in self.groups])
        self.padding_slot = max_slots
        self._states: Dict[int, torch.Tensor] = {}
        for cid, req in state_requests.items():
            if req is not None:
                self._states[cid] = torch.zeros((max_slots + 1, *req.shape), dtype=req.dtype, device=device)
        # sampler state: one xorshift64* word per slot
        self.rng_states = torch.zeros(max_slots + 1, dtype=torch.int64, device=device)
        # the token sampled last for the sequence of each slot: the next step's input can be read
        # from here on the device (token id -1) before the host has seen it
        self.last_token = torch.zeros(max_slots + 1, dtype=torch.int32, device=device)

    # ---- views -----------------------------------------------------------------
    def view(self, cache_id: int) -> Optional[CacheView]:
        return self._views.get(cache_id)

    def state(self, cache_id: int) -> Optional[torch.Tensor]:
        return self._states.get(cache_id)

    def bytes(self) -> int:
        return sum(g.bytes() for g in self.groups)

    # ---- slots -----------------------------------------------------------------
    def acquire(self) -> int:
        s = self.ledger.acquire()
        for t in self._states.values():
            t[s].zero_()
        return s

    def release(self, slot: int) -> None:
        self.ledger.release(slot)

    def length(self, slot: int) -> int:
        return self.ledger.length[slot]

    def truncate(self, slot: int, new_length: int) -> None:
        """Forget the tokens of ``slot`` from ``new_length`` on.  Keys and values are simply written
        over by what comes next; state of fixed size cannot be taken back, so a cache that holds any
        refuses a rewind (a mixer that wants it has to keep snapshots of its own)."""
        if self._states and new_length < self.length(slot):
            raise CacheError("this model keeps per-sequence state of fixed size, which cannot be rewound")
        self.ledger.truncate(slot, new_length, [g.window or 0 for g in self.groups])
