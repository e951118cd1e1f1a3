"""The description of one step that every part receives.

A step runs ``num_tokens`` tokens of ``num_seqs`` sequences as one batch.  Tokens
of a sequence are contiguous; ``cu_seqlens`` delimits them.  All index tensors
are int32 on the device and are slices of ONE buffer that is filled on the host
and copied once.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch


@dataclass
class StepBatch:
    num_tokens: int
    num_seqs: int
    num_want: int
    token_ids: torch.Tensor      # [T]   token id
    seq_of_token: torch.Tensor   # [T]   index into the per-sequence arrays, -1 for a padding row
    pos: torch.Tensor            # [T]   position of the token in its sequence
    cu_seqlens: torch.Tensor     # [B+1] first token of each sequence
    slots: torch.Tensor          # [B]   cache slot of each sequence
    seq_start: torch.Tensor      # [B]   length of the sequence before this step
    seq_end: torch.Tensor        # [B]   ... and after it
    want_rows: torch.Tensor      # [W]   token rows whose logits are wanted
    # host-side facts that choose kernels and size grids
    max_new: int = 0             # most tokens any sequence brings
    max_end: int = 0             # longest sequence after the step
    all_decode: bool = False     # every sequence brings exactly one token
    all_fresh: bool = False      # every sequence starts at position 0


def layout(num_tokens: int, num_seqs: int, num_want: int) -> List[Tuple[str, int]]:
    return [
        ("token_ids", num_tokens), ("seq_of_token", num_tokens), ("pos", num_tokens),
        ("cu_seqlens", num_seqs + 1), ("slots", num_seqs), ("seq_start", num_seqs), ("seq_end", num_seqs),
        ("want_rows", max(num_want, 1)),
    ]


def fill_host(buf: np.ndarray, slots: Sequence[int], starts: Sequence[int], tokens: Sequence[Sequence[int]],
              want: Sequence[Sequence[int]]) -> dict:
    """Write the step's index arrays into ``buf`` (int32); return name -> (offset, length)
    plus the host-side facts."""
    B = len(slots)
    counts = [len(t) for t in tokens]
    T = sum(counts)
    W = sum(len(w) for w in want)
    offs, o = {}, 0
    for name, n in layout(T, B, W):
        offs[name] = (o, n)
        o += n
    if o > buf.size:
        raise ValueError("staging buffer too small")
    v = {k: buf[a:a + n] for k, (a, n) in offs.items()}
    cu = 0
    wi = 0
    for s in range(B):
        n = counts[s]
        v["token_ids"][cu:cu + n] = tokens[s]
        v["seq_of_token"][cu:cu + n] = s
        v["pos"][cu:cu + n] = np.arange(starts[s], starts[s] + n, dtype=np.int32)
        v["cu_seqlens"][s] = cu
        v["slots"][s] = slots[s]
        v["seq_start"][s] = starts[s]
        v["seq_end"][s] = starts[s] + n
        for w in want[s]:
            if not 0 <= w < n:
                raise ValueError(f"wanted place {w} is not among the {n} tokens of this step")
            v["want_rows"][wi] = cu + w
            wi += 1
        cu += n
    v["cu_seqlens"][B] = cu
    if W == 0:
        v["want_rows"][0] = 0
    facts = dict(
        num_tokens=T, num_seqs=B, num_want=W, max_new=max(counts), max_end=max(s + n for s, n in zip(starts, counts)),
        all_decode=all(n == 1 for n in counts), all_fresh=all(s == 0 for s in starts),
    )
    return {"offsets": offs, "used": o, "facts": facts}
