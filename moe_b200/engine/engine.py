"""The step function: a model, its cache, and one call that runs a batch of tokens.

``Engine.step`` takes, for each sequence of the batch, its slot, its next tokens
and the places among them whose logits are wanted.  It appends to the cache and
returns the float32 logits of the wanted places, in the order given.  Sequences
may bring different numbers of tokens; a result does not depend on what else is
in the batch (reference: one sequence per call, src/model.rs:565-589; prefill
and decode are the same code there too).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..cache.allocator import CacheError, pages_for
from ..cache.kv import KVCache
from ..models.decoder import DecoderModel
from ..ops import core
from .batch import StepBatch, fill_host


class Engine:
    def __init__(self, model: DecoderModel, max_tokens: int, max_slots: Optional[int] = None):
        self.model = model
        self.rt = model.rt
        if self.rt.device.type != "cuda":
            raise RuntimeError("the engine runs on a CUDA device; there is no CPU path")
        core.lib()   # fail now, loudly, if the kernels cannot be built or loaded
        if max_slots is None:
            max_slots = max(1, min(1024, -(-max_tokens // 64)))
        self.cache = KVCache(model.kv_requests(), model.state_requests(), max_tokens, max_slots,
                             self.rt.compute_dtype, self.rt.device)
        self.vocab_size = model.spec.vocab_size
        self._stage_host: Optional[torch.Tensor] = None
        self._stage_dev: Optional[torch.Tensor] = None
        self._stage_event = torch.cuda.Event()
        self._stage_busy = False
        self.steps_run = 0

    # ---- sequences -----------------------------------------------------------------
    def new_sequence(self) -> int:
        return self.cache.acquire()

    def release(self, slot: int) -> None:
        self.cache.release(slot)

    def length(self, slot: int) -> int:
        return self.cache.length(slot)

    # ---- staging ---------------------------------------------------------------------
    def _staging(self, n: int) -> Tuple[np.ndarray, torch.Tensor]:
        if self._stage_busy:
            self._stage_event.synchronize()
            self._stage_busy = False
        if self._stage_host is None or self._stage_host.numel() < n:
            size = max(4096, 1 << (n - 1).bit_length())
            self._stage_host = torch.empty(size, dtype=torch.int32).pin_memory()
            self._stage_dev = torch.empty(size, dtype=torch.int32, device=self.rt.device)
        return self._stage_host.numpy(), self._stage_dev

    # ---- the step ----------------------------------------------------------------------
    def _reserve(self, slots: Sequence[int], counts: Sequence[int]) -> List[Tuple[int, int, int, int]]:
        """Give every sequence room for its new tokens, or change nothing and raise."""
        led = self.cache.ledger
        if len(set(slots)) != len(slots):
            raise ValueError("a slot appears twice in one step")
        need = [0] * len(led.groups)
        for s, n in zip(slots, counts):
            if not led.slots.is_held(s):
                raise CacheError(f"slot {s} is not held")
            if n <= 0:
                raise ValueError("every sequence of a step brings at least one token")
            for gi, g in enumerate(led.groups):
                need[gi] += max(0, pages_for(led.length[s] + n, g.ring_pages) - len(g.pages[s]))
        for gi, g in enumerate(led.groups):
            if need[gi] > g.pool.num_free:
                raise CacheError(
                    f"the cache is full: this step needs {need[gi]} more pages of 64 tokens, "
                    f"{g.pool.num_free} are free (max_tokens = {self.cache.max_tokens})"
                )
            if not g.ring_pages:
                for s, n in zip(slots, counts):
                    if pages_for(led.length[s] + n) > self.cache.groups[gi].max_pages_per_seq:
                        raise CacheError("a sequence would outgrow the page table")
        updates = []
        for s, n in zip(slots, counts):
            updates.extend(led.extend(s, led.length[s] + n))
        return updates

    def step(self, slots: Sequence[int], tokens: Sequence[Sequence[int]],
             want: Optional[Sequence[Sequence[int]]] = None, check: bool = True) -> Optional[torch.Tensor]:
        """Run ``tokens[i]`` for the sequence in ``slots[i]``; return logits at ``want[i]``.

        ``want[i]`` lists places among ``tokens[i]`` (0 = its first token of this
        step); by default the last place of each sequence.  The result is a float32
        CUDA tensor [sum(len(w)), vocab], or None if nothing is wanted."""
        B = len(slots)
        if B == 0:
            return None
        if len(tokens) != B:
            raise ValueError("slots and tokens differ in length")
        if want is None:
            want = [[len(t) - 1] for t in tokens]
        counts = [len(t) for t in tokens]
        if len(want) != B:
            raise ValueError("slots and want differ in length")
        for n, w in zip(counts, want):
            for i in w:
                if not 0 <= i < n:
                    raise ValueError(f"wanted place {i} is not among the {n} tokens of this step")
        starts = [self.cache.length(s) if self.cache.ledger.slots.is_held(s) else 0 for s in slots]
        updates = self._reserve(slots, counts)
        T, W = sum(counts), sum(len(w) for w in want)
        n_upd = len(updates)
        host, dev = self._staging(3 * T + 4 * B + 2 + max(W, 1) + 3 * n_upd)
        info = fill_host(host, slots, starts, tokens, want)
        used = info["used"]
        upd_off: Dict[int, Tuple[int, int]] = {}
        if n_upd:
            o = used
            for gi in range(len(self.cache.groups)):
                mine = [(s, i, p) for g, s, i, p in updates if g == gi]
                if mine:
                    host[o:o + 3 * len(mine)] = np.asarray(mine, dtype=np.int32).reshape(-1)
                    upd_off[gi] = (o, len(mine))
                    o += 3 * len(mine)
            used = o
        dev[:used].copy_(self._stage_host[:used], non_blocking=True)
        self._stage_event.record()
        self._stage_busy = True
        for gi, (o, n) in upd_off.items():
            core.table_update(self.cache.groups[gi].table, dev[o:o + 3 * n], n)
        views = {k: dev[a:a + n] for k, (a, n) in info["offsets"].items()}
        batch = StepBatch(**views, **info["facts"])
        self.last_batch = batch
        logits = self.model.forward(batch, self.cache)
        self.steps_run += 1
        if check:
            self.rt.check()
        return logits

    def step_and_sample(self, slots: Sequence[int], tokens: Sequence[Sequence[int]], sampler, params,
                        histories=None) -> List[int]:
        """One step, then one sampled token per sequence from the logits at its last
        place; tokens come back to the host (one small copy, which also carries the
        device status word)."""
        logits = self.step(slots, tokens, None, check=False)
        picked = sampler.sample(logits, self.last_batch.slots, params, histories)
        host = torch.cat([picked, self.rt.status[:1]]).cpu()
        if int(host[-1]):
            self.rt.check()
        return host[:-1].tolist()
