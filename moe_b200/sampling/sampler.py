"""Sampling on the device: one kernel call per step for the whole batch.

The random-number state of a sequence (xorshift64*, src/sample.rs:4-19) lives in
the cache's fixed-size state area, indexed by the sequence's slot, so that it
follows the sequence through batches of any composition.
"""
from __future__ import annotations

from typing import Optional, Sequence

import numpy as np
import torch

from ..ops import core
from .params import SamplingParams


class DeviceSampler:
    def __init__(self, rng_states: torch.Tensor, device, last_token: Optional[torch.Tensor] = None):
        self.rng_states = rng_states
        self.device = device
        self.last_token = last_token     # per-slot table that also receives every sampled token

    def seed(self, slots: Sequence[int], seeds: Sequence[int]) -> None:
        """state = seed * 0x9e3779b97f4a7c15 | 1 for each slot (src/sample.rs:7-9)."""
        s = torch.tensor(list(slots), dtype=torch.int32, device=self.device)
        v = np.asarray([x & 0xFFFFFFFFFFFFFFFF for x in seeds], dtype=np.uint64).view(np.int64)
        core.seed_rng(self.rng_states, s, torch.from_numpy(v.copy()).to(self.device))

    def history_tensor(self, histories: Sequence[Sequence[int]], window: int) -> Optional[torch.Tensor]:
        """[rows, window] int32, most recent first, -1 padded."""
        if window <= 0:
            return None
        h = np.full((len(histories), window), -1, dtype=np.int32)
        for i, hist in enumerate(histories):
            tail = list(hist[-window:])[::-1]
            h[i, :len(tail)] = tail
        return torch.from_numpy(h).to(self.device)

    def sample(self, logits: torch.Tensor, slots: torch.Tensor, params: SamplingParams,
               histories: Optional[Sequence[Sequence[int]]] = None,
               out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """logits: [rows, vocab] float32 (modified in place by a repeat penalty);
        slots: int32 [rows] on the device.  Returns int32 [rows] on the device."""
        rows = logits.shape[0]
        if out is None:
            out = torch.empty(rows, dtype=torch.int32, device=logits.device)
        hist = None
        if params.repeat_penalty != 1.0 and histories is not None:
            hist = self.history_tensor(histories, params.repeat_window)
        core.sample(logits, slots, self.rng_states, out, temp=params.temp, top_k=params.top_k, top_p=params.top_p,
                    repeat_penalty=params.repeat_penalty if hist is not None else 1.0, history=hist,
                    last_token=self.last_token)
        return out
