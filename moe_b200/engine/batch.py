"""The description of one step that every part receives.

A step runs ``num_tokens`` tokens of ``num_seqs`` sequences as one batch.  Tokens
of a sequence are contiguous; ``cu_seqlens`` delimits them.  All index tensors
are int32 on the device and are slices of ONE buffer that is filled on the host
and copied once.
"""
from __future__ import annotations

import ctypes
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
    # per-slot table of the tokens sampled last; if given, a token id of -1 is read from it
    last_token: Optional[torch.Tensor] = None
    # a step of several tokens a sequence with rows that belong to no sequence (a padded graph): a
    # mixer must leave something finite in those rows of its output, as rows of a tile are multiplied
    # by weights of exactly zero, and 0 x NaN is NaN
    has_padding: bool = False


def layout(num_tokens: int, num_seqs: int, num_want: int) -> List[Tuple[str, int]]:
    return [
        ("token_ids", num_tokens), ("seq_of_token", num_tokens), ("pos", num_tokens),
        ("cu_seqlens", num_seqs + 1), ("slots", num_seqs), ("seq_start", num_seqs), ("seq_end", num_seqs),
        ("want_rows", max(num_want, 1)),
    ]


def fill_host(buf: np.ndarray, slots: Sequence[int], starts: Sequence[int], tokens: Sequence[Sequence[int]],
              want: Sequence[Sequence[int]]) -> dict:
    """Write the step's index arrays into ``buf`` (int32, C-contiguous); return name ->
    (offset, length) plus the host-side facts.  The packing itself is the host runtime's
    ``moe_pack_step`` (``csrc/host_runtime.cpp``)."""
    from ..cache.allocator import _IP, _ok, host_lib, ints

    L = host_lib()
    B = len(slots)
    counts = [len(t) for t in tokens]
    flat = np.fromiter((x for t in tokens for x in t), dtype=np.int32, count=sum(counts))
    wflat = np.fromiter((x for w in want for x in w), dtype=np.int32, count=sum(len(w) for w in want))
    sl, _ = ints(slots)
    st, _ = ints(starts)
    ct, _ = ints(counts)
    wc, _ = ints([len(w) for w in want])
    offs = (ctypes.c_int * 8)()
    facts = (ctypes.c_int * 7)()
    used = L.moe_pack_step(buf.ctypes.data_as(_IP), buf.size, B, sl, st, ct, flat.ctypes.data_as(_IP), wc,
                           wflat.ctypes.data_as(_IP), offs, facts)
    _ok(int(used))
    T, _, W = facts[0], facts[1], facts[2]
    names = [n for n, _ in layout(T, B, W)]
    sizes = [n for _, n in layout(T, B, W)]
    return {
        "offsets": {n: (offs[i], sizes[i]) for i, n in enumerate(names)},
        "used": int(used),
        "facts": dict(num_tokens=T, num_seqs=B, num_want=W, max_new=facts[3], max_end=facts[4],
                      all_decode=bool(facts[5]), all_fresh=bool(facts[6])),
    }
