"""Architecture-independent description of a decoder, layer by layer.

An architecture's typed configuration is translated once into a ``ModelSpec``:
a list of layers, each naming the kind and the constants of its parts, plus the
order in which layers run.  Everything downstream (weight checking, random
initialisation, the cache, the engine) works from the ``ModelSpec`` alone and
never asks which architecture produced it.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple


@dataclass(frozen=True)
class PartSpec:
    """One part of a layer: which implementation (``kind``) and its constants.

    ``prefix`` is prepended to the part's local tensor names to form checkpoint
    names, e.g. ``model.layers.3.self_attn.``.
    """

    kind: str
    params: Dict[str, Any] = field(default_factory=dict)
    prefix: str = ""


@dataclass(frozen=True)
class LayerSpec:
    """A block: how a mixer, a feed-forward and their norms are arranged."""

    block: str            # registered block arrangement, e.g. "prenorm"
    norm1: PartSpec
    mixer: PartSpec
    norm2: PartSpec
    ffn: PartSpec


@dataclass(frozen=True)
class ScheduleEntry:
    """One run of a layer inside a step.

    ``layer`` indexes ``ModelSpec.layers``.  ``cache`` names the cache entry the
    mixer uses; two entries with the same ``cache`` share keys and values, and
    only the one with ``writes_cache`` appends to it.
    """

    layer: int
    cache: int
    writes_cache: bool = True


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    hidden_size: int
    vocab_size: int
    embedding: PartSpec
    layers: Tuple[LayerSpec, ...]
    schedule: Tuple[ScheduleEntry, ...]
    final_norm: PartSpec
    head: PartSpec
    eos_token_ids: Tuple[int, ...] = ()
    bos_token_id: Optional[int] = None
    max_position_embeddings: Optional[int] = None
    # checkpoint names that may be present but carry no weight of the model
    ignorable: Tuple[str, ...] = ()

    def cache_entries(self) -> List[int]:
        seen: List[int] = []
        for e in self.schedule:
            if e.cache not in seen:
                seen.append(e.cache)
        return seen
