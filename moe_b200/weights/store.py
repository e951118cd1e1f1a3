"""Weights addressed by tensor name.

A ``WeightStore`` answers three questions: which names exist, what shape and
stored dtype each has, and the tensor itself.  ``check`` compares a model's
expected tensors with what the store holds and raises ONE error that lists
everything missing, unexpected or wrongly shaped (the reference stops at the
first missing tensor, src/model.rs:342).

Dtype policy when a tensor is handed to a part:
  * compute dtype float32: every floating tensor is widened exactly to float32
    (bf16 -> f32 is ``bits << 16``, src/quant.rs:189-193);
  * compute dtype bfloat16: a tensor stored in bfloat16 stays bfloat16, a tensor
    stored in 32-bit stays 32-bit, float16 is widened to float32 (exact);
  * integer tables become int32.
"""
from __future__ import annotations

import fnmatch
from typing import Dict, Iterable, List, Tuple

import torch

from .safetensors_io import SafetensorsError, SafetensorsFile, shard_paths


class WeightError(ValueError):
    """Missing, unexpected or wrongly shaped tensors; all of them in one message."""

    def __init__(self, missing, unexpected, wrong_shape, wrong_dtype=()):
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        self.wrong_dtype = list(wrong_dtype)
        lines = ["the weights do not match the configuration:"]
        if self.missing:
            lines.append(f"  missing ({len(self.missing)}): " + _abbrev(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected ({len(self.unexpected)}): " + _abbrev(self.unexpected))
        if self.wrong_shape:
            lines.append(
                f"  wrong shape ({len(self.wrong_shape)}): "
                + _abbrev([f"{n} is {list(g)}, expected {list(e)}" for n, g, e in self.wrong_shape])
            )
        if self.wrong_dtype:
            lines.append(
                f"  wrong dtype ({len(self.wrong_dtype)}): " + _abbrev([f"{n} is {d}" for n, d in self.wrong_dtype])
            )
        super().__init__("\n".join(lines))


def _abbrev(items: List[str], limit: int = 24) -> str:
    if len(items) <= limit:
        return ", ".join(items)
    return ", ".join(items[:limit]) + f", ... and {len(items) - limit} more"


_FLOATS = (torch.float32, torch.float16, torch.bfloat16, torch.float64)


def convert_for_compute(t: torch.Tensor, compute_dtype: torch.dtype) -> torch.Tensor:
    if t.dtype in _FLOATS:
        if compute_dtype == torch.float32:
            return t.to(torch.float32)
        if t.dtype == torch.bfloat16:
            return t
        return t.to(torch.float32)
    if t.dtype == torch.bool:
        return t
    return t.to(torch.int32)


class WeightStore:
    """Interface; see ``SafetensorsStore`` and ``TensorDictStore``."""

    def names(self) -> Iterable[str]:
        raise NotImplementedError

    def shape(self, name: str) -> Tuple[int, ...]:
        raise NotImplementedError

    def stored_dtype(self, name: str) -> torch.dtype:
        raise NotImplementedError

    def raw(self, name: str) -> torch.Tensor:
        raise NotImplementedError

    def has(self, name: str) -> bool:
        return name in set(self.names())

    def get(self, name: str, compute_dtype: torch.dtype, device="cpu") -> torch.Tensor:
        """The tensor under the dtype policy, on ``device``, contiguous and owned."""
        t = convert_for_compute(self.raw(name), compute_dtype)
        t = t.to(device=device, copy=True) if str(device) == "cpu" else t.to(device=device)
        return t.contiguous()

    def check(self, expected: Dict[str, Tuple[int, ...]], ignorable: Iterable[str] = ()) -> None:
        have = set(self.names())
        missing = sorted(n for n in expected if n not in have)
        patterns = list(ignorable)
        unexpected = sorted(
            n for n in have if n not in expected and not any(fnmatch.fnmatchcase(n, p) for p in patterns)
        )
        wrong, wrong_dt = [], []
        for n, shp in expected.items():
            if n in have:
                if tuple(self.shape(n)) != tuple(shp):
                    wrong.append((n, tuple(self.shape(n)), tuple(shp)))
                if self.stored_dtype(n) not in _FLOATS:
                    wrong_dt.append((n, str(self.stored_dtype(n))))
        if missing or unexpected or wrong or wrong_dt:
            raise WeightError(missing, unexpected, sorted(wrong), sorted(wrong_dt))


class SafetensorsStore(WeightStore):
    """Every ``*.safetensors`` shard of a folder, sorted; a later shard wins on a
    duplicate name (src/store.rs:182-197)."""

    def __init__(self, model_dir: str):
        self.model_dir = model_dir
        self.files = [SafetensorsFile(p, i) for i, p in enumerate(shard_paths(model_dir))]
        self.index = {}
        for f in self.files:
            self.index.update(f.records)

    def names(self):
        return self.index.keys()

    def has(self, name):
        return name in self.index

    def shape(self, name):
        return self.index[name].shape

    def stored_dtype(self, name):
        return self.raw_dtype(name)

    def raw_dtype(self, name):
        from .safetensors_io import _DTYPES

        return _DTYPES[self.index[name].dtype][0]

    def raw(self, name):
        rec = self.index.get(name)
        if rec is None:
            raise SafetensorsError(f"missing tensor: {name}")
        return self.files[rec.file].tensor(rec)


class TensorDictStore(WeightStore):
    """Tensors already in memory (on any device), e.g. freshly drawn random weights."""

    def __init__(self, tensors: Dict[str, torch.Tensor]):
        self.tensors = tensors

    def names(self):
        return self.tensors.keys()

    def has(self, name):
        return name in self.tensors

    def shape(self, name):
        return tuple(self.tensors[name].shape)

    def stored_dtype(self, name):
        return self.tensors[name].dtype

    def raw(self, name):
        return self.tensors[name]

    def get(self, name, compute_dtype, device="cpu"):
        t = convert_for_compute(self.tensors[name], compute_dtype)
        return t.to(device=device).contiguous()
