"""Helpers of the GPU tests: engines per configuration, hand-made step batches."""
from __future__ import annotations

from typing import Dict, Optional, Sequence

import numpy as np
import torch

import helpers

# Tolerances, relative to the largest logit of the reference (max |got - ref| / max |ref|).
#   float32 path against the plain float64 implementation: accumulation order only.
#   bfloat16 path: inputs of every matrix product, queries and the cache are rounded to 8 bits
#   of mantissa (unit roundoff u = 2^-9 = 2e-3); a few such roundings per layer give 2-5 u on
#   a model whose matrices have gain <= 1.  Random weights of std 0.2 have gain 1.6 per matrix
#   at these widths and amplify any perturbation 10-20 times from embedding to logits (measured:
#   4e-3 at std <= 0.08, 1e-2 at 0.125, 5e-2 at 0.2, the 32-bit path staying below 5e-6
#   throughout), so bfloat16 is compared on std 0.02 and 0.08 and 32-bit on 0.02 and 0.2.
TOL_F32 = 5e-5
TOL_BF16 = 2e-2
STD = {"float32": (0.02, 0.2), "bfloat16": (0.02, 0.08)}
# for the configuration that is 264 wide (and whose heads are 128 long, so its sums are longer too): the
# same gain per matrix, std * sqrt(width), as 0.2 / 0.08 give at a width of 96
STD_WIDE = {"float32": 0.12, "bfloat16": 0.048}
# The same tokens cut differently (whole / one by one / batched), same dtype.
TOL_CUT_F32 = 1e-5
TOL_CUT_BF16 = 1e-2
# A routing pick may differ from the plain implementation's only where the two experts' router
# logits are this close, as a fraction of the root mean square of the layer's router logits
# (``helpers.pick_margins``).  An error of relative size eps in the normed state moves a logit by
# about eps of that scale, and the difference of two by sqrt(2) eps; with eps = 1e-2 for bfloat16
# (half of TOL_BF16, the bound on what the same error leaves in the output logits) a three-sigma
# event among the thousands of picks a test makes is 3 sqrt(2) eps = 4.2e-2.  In float32, eps = 2.5e-5.
FLIP_F32 = 1e-4
FLIP_BF16 = 4.5e-2

_engines: Dict[tuple, object] = {}


def engine_for(model_dirs, name: str, dtype: str, std: Optional[float] = None, seed: int = 1, max_tokens: int = 2048,
               max_slots: Optional[int] = None, overrides=None):
    """(model folder, engine), cached for the session.  ``std`` defaults to the larger of the
    dtype's two weight scales."""
    import moe_b200
    from moe_b200.engine import Engine

    if std is None:
        std = STD_WIDE[dtype] if helpers.CONFIGS[name]["hidden_size"] > 200 else STD[dtype][1]

    d = model_dirs.get(name, dtype, seed=seed, std=std, overrides=overrides)
    key = (d, dtype, max_tokens, max_slots)
    if key not in _engines:
        _engines[key] = Engine(moe_b200.load_model(d, dtype=dtype), max_tokens=max_tokens, max_slots=max_slots)
    return d, _engines[key]


def tol(dtype: str) -> float:
    return TOL_F32 if dtype == "float32" else TOL_BF16


def tol_cut(dtype: str) -> float:
    return TOL_CUT_F32 if dtype == "float32" else TOL_CUT_BF16


def flip(dtype: str) -> float:
    return FLIP_F32 if dtype == "float32" else FLIP_BF16


def make_batch(device, slots: Sequence[int], starts: Sequence[int], counts: Sequence[int],
               tokens: Optional[Sequence[Sequence[int]]] = None, want=None):
    """A StepBatch for calling kernels and parts directly."""
    from moe_b200.engine.batch import StepBatch, fill_host

    tokens = tokens or [[0] * n for n in counts]
    want = want or [[] for _ in counts]
    host = np.zeros(3 * sum(counts) + 4 * len(slots) + 8 + sum(len(w) for w in want), dtype=np.int32)
    info = fill_host(host, slots, starts, tokens, want)
    dev = torch.from_numpy(host).to(device)
    views = {k: dev[a:a + n] for k, (a, n) in info["offsets"].items()}
    return StepBatch(**views, **info["facts"])


def give_pages(cache, slot: int, length: int):
    """Reserve pages for ``length`` tokens of ``slot`` and write them into the device tables."""
    from moe_b200.ops import core

    for gi, s, i, p in cache.ledger.extend(slot, length):
        upd = torch.tensor([s, i, p], dtype=torch.int32, device=cache.device)
        core.table_update(cache.groups[gi].table, upd, 1)
