"""A decoder assembled from a ``ModelSpec``: embedding, blocks run in the order
of the schedule, final norm and output projection (src/model.rs:646-687, 637-643).

Nothing here names an architecture; the spec says which parts each layer has.
"""
from __future__ import annotations

from collections.abc import Mapping
from typing import Dict, List, Optional

import torch

from ..cache.kv import KVRequest, StateRequest
from ..config.spec import ModelSpec
from ..parts import block as block_mod
from ..parts.base import Part, Runtime, TensorSpec, delta_for, make_part
from ..weights.store import WeightStore


def _named_parts(spec: ModelSpec):
    """Yield (part, prefix) for every part of the model, unbound."""
    emb = make_part("embedding", spec.embedding)
    blocks = [block_mod.make_block(l) for l in spec.layers]
    final_norm = make_part("norm", spec.final_norm)
    head = make_part("head", spec.head)
    return emb, blocks, final_norm, head


class PartTensors(Mapping):
    """The tensors of one part, by local name, fetched from the store when they are asked for and
    not kept: a part that re-lays its weights out (one slab for all experts, say) holds a tensor of
    the store only while it copies it.  ``pop`` is a fetch too."""

    def __init__(self, store: WeightStore, prefix: str, names, dtype, device):
        self._store, self._prefix, self._names = store, prefix, list(names)
        self._dtype, self._device = dtype, device

    def __getitem__(self, local):
        if local not in self._names:
            raise KeyError(local)
        return self._store.get(self._prefix + local, self._dtype, self._device)

    def pop(self, local, *default):
        if local not in self._names and default:
            return default[0]
        return self[local]

    def __iter__(self):
        return iter(self._names)

    def __len__(self):
        return len(self._names)


def _tensors_of(part: Part, store: Optional[WeightStore]) -> Dict[str, TensorSpec]:
    if store is None:
        return part.tensors()
    return part.tensors_in(lambda local: store.has(part.spec.prefix + local))


def expected_tensors(spec: ModelSpec, store: Optional[WeightStore] = None) -> Dict[str, TensorSpec]:
    """Checkpoint name -> shape of every tensor the model needs; with a ``store``, in the layout
    that each part finds there (a part may take several, ``Part.tensors_in``)."""
    emb, blocks, final_norm, head = _named_parts(spec)
    out: Dict[str, TensorSpec] = {}
    parts: List[Part] = [emb, final_norm, head]
    for b in blocks:
        parts.extend(b.parts())
    for p in parts:
        for local, ts in _tensors_of(p, store).items():
            out[p.spec.prefix + local] = ts
    return out


class DecoderModel:
    def __init__(self, spec: ModelSpec, store: WeightStore, rt: Runtime, check: bool = True):
        self.spec = spec
        self.rt = rt
        self.embedding, self.blocks, self.final_norm, self.head = _named_parts(spec)
        if check:
            store.check({n: ts.shape for n, ts in expected_tensors(spec, store).items()}, spec.ignorable)
        self._validate_schedule()

        def bind(part: Part, **kw):
            part.bind(PartTensors(store, part.spec.prefix, _tensors_of(part, store), rt.compute_dtype, rt.device),
                      rt, **kw)

        bind(self.embedding)
        for b in self.blocks:
            for p in b.parts():
                bind(p)
        bind(self.final_norm)
        bind(self.head, embedding=self.embedding)
        self.num_parameters = sum(
            int(torch.tensor(ts.shape).prod()) for ts in expected_tensors(spec).values()
        )

    # ---- cache needs -------------------------------------------------------------
    def _validate_schedule(self):
        writers: Dict[int, int] = {}
        for i, e in enumerate(self.spec.schedule):
            if not 0 <= e.layer < len(self.blocks):
                raise ValueError(f"schedule entry {i} names layer {e.layer} of {len(self.blocks)}")
            mixer = self.blocks[e.layer].mixer
            own = getattr(mixer, "own_kv", True)
            if e.writes_cache:
                if e.cache in writers:
                    raise ValueError(f"cache entry {e.cache} is written by schedule entries {writers[e.cache]} and {i}")
                if not own:
                    raise ValueError(f"schedule entry {i} writes cache {e.cache} but its mixer projects no keys")
                writers[e.cache] = i
            else:
                if e.cache not in writers:
                    raise ValueError(f"schedule entry {i} reads cache {e.cache} before any entry wrote it")
                if own:
                    raise ValueError(f"schedule entry {i} reads another layer's cache but its mixer has keys of its own")
                a = mixer.kv_request()
                b = self.blocks[self.spec.schedule[writers[e.cache]].layer].mixer.kv_request()
                if a != b:
                    raise ValueError(f"schedule entry {i} reads cache {e.cache} with a different record shape")

    def kv_requests(self) -> Dict[int, Optional[KVRequest]]:
        out: Dict[int, Optional[KVRequest]] = {}
        for e in self.spec.schedule:
            if e.writes_cache:
                out[e.cache] = self.blocks[e.layer].mixer.kv_request()
        return out

    def state_requests(self) -> Dict[int, Optional[StateRequest]]:
        out: Dict[int, Optional[StateRequest]] = {}
        for e in self.spec.schedule:
            if e.writes_cache:
                out[e.cache] = self.blocks[e.layer].mixer.state_request()
        return out

    # ---- one step ------------------------------------------------------------------
    def forward(self, batch, cache) -> Optional[torch.Tensor]:
        """Run the batch's tokens through every scheduled layer, appending to the cache;
        return float32 logits [len(want_rows), vocab], or None if no row is wanted."""
        rt = self.rt
        x = self.embedding.forward(rt, batch.token_ids, batch.num_tokens, batch)
        pending = None
        for e in self.spec.schedule:
            x, pending = self.blocks[e.layer].forward(rt, x, pending, batch, cache.view(e.cache), cache.state(e.cache))
        if batch.num_want == 0:
            return None
        h = self.final_norm.forward(rt, x, delta=delta_for(self.final_norm, pending, rt), rows=batch.want_rows,
                                    write_back=False)
        return self.head.forward(rt, h)
