"""One registry from an architecture's name to its configuration and model.

The reference engine detects what a checkpoint is from its tensors
(src/model.rs:341-480, src/spec.rs:245-339).  Here the name in config.json
(``architectures[0]``, else ``model_type``; src/spec.rs:310-314) selects a
registered entry, and an unknown name is an error that lists what is known.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Any, Callable, Dict

from .spec import ModelSpec


class ConfigError(ValueError):
    """A config.json that cannot describe a model of its architecture."""


@dataclass(frozen=True)
class Architecture:
    name: str
    parse_config: Callable[[Dict[str, Any]], Any]      # dict -> typed config
    model_spec: Callable[[Any], ModelSpec]             # typed config -> ModelSpec
    config_dict: Callable[[Any], Dict[str, Any]]       # typed config -> config.json dict


_ARCHITECTURES: Dict[str, Architecture] = {}
_ALIASES: Dict[str, str] = {}


def register_architecture(arch: Architecture, *, model_types: tuple = ()) -> None:
    _ARCHITECTURES[arch.name] = arch
    for t in model_types:
        _ALIASES[t] = arch.name


def registered_architectures() -> list:
    return sorted(_ARCHITECTURES)


def architecture_name(config: Dict[str, Any]) -> str:
    archs = config.get("architectures")
    if isinstance(archs, list) and archs and isinstance(archs[0], str):
        return archs[0]
    mt = config.get("model_type")
    if isinstance(mt, str):
        return _ALIASES.get(mt, mt)
    raise ConfigError("config.json names no architecture (neither 'architectures' nor 'model_type')")


def lookup(name: str) -> Architecture:
    name = _ALIASES.get(name, name)
    if name not in _ARCHITECTURES:
        raise ConfigError(
            f"unknown architecture '{name}'; registered: {', '.join(registered_architectures()) or '(none)'}"
        )
    return _ARCHITECTURES[name]


def read_config_json(model_dir: str) -> Dict[str, Any]:
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"{model_dir}: no config.json")
    with open(path, "r", encoding="utf-8") as f:
        try:
            cfg = json.load(f)
        except json.JSONDecodeError as e:
            raise ConfigError(f"{path}: not valid JSON: {e}") from None
    if not isinstance(cfg, dict):
        raise ConfigError(f"{path}: top level must be an object")
    return cfg


def parse_config(config: Dict[str, Any]):
    """config.json dict -> (Architecture, typed config)."""
    arch = lookup(architecture_name(config))
    return arch, arch.parse_config(config)
