"""Random weights from a configuration and a seed.

The reference has no such mode (its tests check in tiny fixtures written by
scripts/oracle.py).  Here every tensor the configuration calls for is drawn
independently from N(0, std) with a generator seeded by (seed, tensor name);
norm weights are 1.  ``write_random_model`` writes a model folder
(config.json, model.safetensors) that loads like any checkpoint.
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Any, Dict, Union

import torch

from ..config import registry
from ..config.spec import ModelSpec
from .safetensors_io import write_safetensors
from .store import WeightStore, convert_for_compute

_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32, "bf16": torch.bfloat16, "fp32": torch.float32,
           torch.bfloat16: torch.bfloat16, torch.float32: torch.float32}


def _tensor_seed(seed: int, name: str) -> int:
    return int.from_bytes(hashlib.sha256(f"{seed}:{name}".encode()).digest()[:7], "little")


def _draw(name: str, ts, seed: int, std: float, dtype, device, norm_jitter: float, gen) -> torch.Tensor:
    gen.manual_seed(_tensor_seed(seed, name))
    if ts.init == "ones":
        t = torch.ones(ts.shape, dtype=torch.float32, device=device)
        if norm_jitter:
            t += norm_jitter * torch.randn(ts.shape, generator=gen, dtype=torch.float32, device=device)
    elif ts.init == "zeros":
        t = torch.zeros(ts.shape, dtype=torch.float32, device=device)
    else:
        t = torch.randn(ts.shape, generator=gen, dtype=torch.float32, device=device) * std
    return t.to(dtype)


def random_tensors(spec: ModelSpec, seed: int, std: float = 0.02, dtype=torch.bfloat16, device="cpu",
                   norm_jitter: float = 0.0) -> Dict[str, torch.Tensor]:
    from ..models.decoder import expected_tensors

    dtype = _DTYPES[dtype]
    gen = torch.Generator(device=device)
    return {name: _draw(name, ts, seed, std, dtype, device, norm_jitter, gen)
            for name, ts in expected_tensors(spec).items()}


class RandomStore(WeightStore):
    """The same random weights, each tensor drawn when it is asked for and kept nowhere: a model
    built from it never holds more than itself and the tensors of the part being bound, which is
    what lets the largest shapes be made on one device.  A tensor's values depend on (seed, name)
    alone, so they equal ``random_tensors``'s drawn on the same kind of device."""

    def __init__(self, spec: ModelSpec, seed: int, std: float = 0.02, dtype=torch.bfloat16, device="cpu",
                 norm_jitter: float = 0.0):
        from ..models.decoder import expected_tensors

        self.expected = expected_tensors(spec)
        self.seed, self.std, self.dtype, self.device, self.norm_jitter = seed, std, _DTYPES[dtype], device, norm_jitter
        self._gen = torch.Generator(device=device)

    def names(self):
        return self.expected.keys()

    def has(self, name):
        return name in self.expected

    def shape(self, name):
        return tuple(self.expected[name].shape)

    def stored_dtype(self, name):
        return self.dtype

    def raw(self, name):
        return _draw(name, self.expected[name], self.seed, self.std, self.dtype, self.device, self.norm_jitter, self._gen)

    def get(self, name, compute_dtype, device="cpu"):
        return convert_for_compute(self.raw(name), compute_dtype).to(device=device).contiguous()


def write_random_model(model_dir: str, config: Union[Dict[str, Any], Any], seed: int, std: float = 0.02,
                       dtype="bfloat16", norm_jitter: float = 0.0) -> str:
    """Write config.json and model.safetensors for ``config`` (a config.json dict or a
    typed configuration) under ``model_dir``; returns the folder."""
    if isinstance(config, dict):
        arch, typed = registry.parse_config(config)
        cfg_dict = dict(config)
    else:
        arch = registry.lookup(getattr(config, "architecture", None) or _arch_of(config))
        typed, cfg_dict = config, arch.config_dict(config)
    spec = arch.model_spec(typed)
    tensors = random_tensors(spec, seed, std, dtype, "cpu", norm_jitter)
    os.makedirs(model_dir, exist_ok=True)
    cfg_dict.setdefault("architectures", [arch.name])
    cfg_dict["torch_dtype"] = "bfloat16" if _DTYPES[dtype] == torch.bfloat16 else "float32"
    with open(os.path.join(model_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(cfg_dict, f, indent=1)
    write_safetensors(os.path.join(model_dir, "model.safetensors"), tensors)
    return model_dir


def _arch_of(typed) -> str:
    for name in registry.registered_architectures():
        a = registry.lookup(name)
        try:
            a.config_dict(typed)
            return name
        except Exception:
            continue
    raise registry.ConfigError(f"no registered architecture takes a {type(typed).__name__}")
