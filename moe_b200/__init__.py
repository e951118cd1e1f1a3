"""moe_b200: a small model library with generation for NVIDIA B200 (sm_100a).

    import moe_b200
    model = moe_b200.load_model("path/to/model", dtype="bfloat16")
    engine = moe_b200.Engine(model, max_tokens=8192)
    out = moe_b200.generate(engine, [[1, 2, 3], [4, 5]], max_tokens=16)
"""
from __future__ import annotations

from typing import Any, Dict, Union

import torch

from . import config as _config  # registers architectures
from . import parts as _parts    # registers parts
from .config import ConfigError, parse_config, read_config_json, register_architecture  # noqa: F401
from .parts import Runtime, register_part  # noqa: F401
from .weights import (RandomStore, SafetensorsStore, TensorDictStore, WeightError, random_tensors,  # noqa: F401
                      write_random_model)

__version__ = "0.1.0"

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
           torch.bfloat16: torch.bfloat16, torch.float32: torch.float32}


def _dtype(dtype) -> torch.dtype:
    if dtype not in _DTYPES:
        raise ValueError(f"dtype must be bfloat16 or float32, not {dtype!r}")
    return _DTYPES[dtype]


def load_model(model_dir: str, dtype="bfloat16", device="cuda"):
    """Load a model folder (config.json + *.safetensors); the class of model is chosen
    by config.json through the architecture registry."""
    from .models import DecoderModel

    arch, typed = parse_config(read_config_json(model_dir))
    spec = arch.model_spec(typed)
    model = DecoderModel(spec, SafetensorsStore(model_dir), Runtime(device, _dtype(dtype)))
    model.config = typed
    return model


def random_model(config: Union[Dict[str, Any], Any], seed: int = 0, dtype="bfloat16", device="cuda",
                 std: float = 0.02, stored_dtype=None):
    """A model with random weights drawn on ``device`` (no files written), part by part: at no
    time is more held than the model itself and the tensors of the part being bound.
    ``stored_dtype``: the dtype the weights are drawn in, as if a checkpoint of that dtype were read
    (default: ``dtype``); a float32 model of bfloat16 weights has exactly the weights of the
    bfloat16 model of the same seed."""
    from .models import DecoderModel

    if isinstance(config, dict):
        arch, typed = parse_config(config)
    else:
        from .weights.random_init import _arch_of

        arch, typed = _config.lookup(_arch_of(config)), config
    spec = arch.model_spec(typed)
    dt = _dtype(dtype)
    model = DecoderModel(spec, RandomStore(spec, seed, std, _dtype(stored_dtype) if stored_dtype else dt, device),
                         Runtime(device, dt), check=False)
    model.config = typed
    return model


def __getattr__(name):
    if name == "Engine":
        from .engine import Engine

        return Engine
    if name == "generate":
        from .api import generate

        return generate
    if name in ("GenerationResult", "GenerationStats"):
        from .engine import generate as _g

        return getattr(_g, name)
    if name == "SamplingParams":
        from .sampling.params import SamplingParams

        return SamplingParams
    raise AttributeError(name)
