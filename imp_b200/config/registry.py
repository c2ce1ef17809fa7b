"""One registry from an architecture's name to its configuration class and model plan.

The reference maps an architecture string to an enum and patches defaults per
family (src/model/model.cpp:70-103), and on the safetensors route guesses the
family from tensor names (src/model/safetensors_loader.cpp:238-263).  Here the
name in config.json's `architectures[0]` selects both the typed configuration
and the function that turns it into a `ModelPlan` (imp_b200/parts/plan.py).
Tests and users add architectures with `register_architecture` without
touching the framework's files.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Any, Callable, Dict, Type

from .model_config import ConfigError, ModelConfig


@dataclass
class ArchitectureEntry:
    name: str
    config_cls: Type[ModelConfig]
    plan_fn: Callable[[ModelConfig], Any]  # -> parts.plan.ModelPlan


_ARCHITECTURES: Dict[str, ArchitectureEntry] = {}


def register_architecture(name: str, config_cls: Type[ModelConfig],
                          plan_fn: Callable[[ModelConfig], Any], *, replace: bool = False) -> None:
    if name in _ARCHITECTURES and not replace:
        raise ValueError(f"architecture '{name}' is already registered")
    _ARCHITECTURES[name] = ArchitectureEntry(name, config_cls, plan_fn)


def unregister_architecture(name: str) -> None:
    _ARCHITECTURES.pop(name, None)


def known_architectures():
    return sorted(_ARCHITECTURES)


def architecture_entry(name: str) -> ArchitectureEntry:
    _ensure_builtin()
    if name not in _ARCHITECTURES:
        raise ConfigError(f"unknown architecture '{name}'; known: {', '.join(known_architectures()) or '(none)'}")
    return _ARCHITECTURES[name]


def _ensure_builtin() -> None:
    # The built-in architectures register themselves on import.
    from .. import architectures  # noqa: F401


def config_from_dict(d: Dict[str, Any], where: str = "config.json") -> ModelConfig:
    archs = d.get("architectures")
    if not archs or not isinstance(archs, list) or not isinstance(archs[0], str):
        raise ConfigError(f"{where}: 'architectures' must be a list that names the model class")
    entry = architecture_entry(archs[0])
    return entry.config_cls.from_json_dict(d, where)


def load_config(model_dir: str) -> ModelConfig:
    path = os.path.join(model_dir, "config.json") if os.path.isdir(model_dir) else model_dir
    if not os.path.exists(path):
        raise ConfigError(f"no config.json at {path}")
    with open(path) as f:
        try:
            d = json.load(f)
        except json.JSONDecodeError as e:
            raise ConfigError(f"{path}: not valid JSON: {e}") from None
    if not isinstance(d, dict):
        raise ConfigError(f"{path}: top level must be an object")
    return config_from_dict(d, path)


def plan_for(config: ModelConfig):
    """The `ModelPlan` (layers, parts, order, tensor names) of a configuration."""
    return architecture_entry(config.architecture).plan_fn(config)
