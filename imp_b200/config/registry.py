"""One registry from an architecture's name to its configuration and model plan.

The registry itself lives in the library (csrc/host/config.cpp); the name in
config.json's `architectures[0]` selects both the typed configuration and the
function that turns it into a plan.  `register_architecture` adds one from
Python: its plan function becomes a callback the library calls with the
config.json text.  The reference maps an architecture string to an enum and
patches defaults per family (src/model/model.cpp:70-103), and on the
safetensors route guesses the family from tensor names
(src/model/safetensors_loader.cpp:238-263).
"""
from __future__ import annotations

import ctypes
import json
import os
from typing import Any, Callable, Dict, Type

from .. import capi
from .model_config import ConfigError, ModelConfig, Qwen3Config

# architectures registered from Python: name -> (config class, plan function, C callback kept alive)
_PY_ARCHS: Dict[str, tuple] = {}
_BUILTIN_CONFIGS: Dict[str, Type[ModelConfig]] = {"Qwen3ForCausalLM": Qwen3Config}


def parse_config_dict(d: Dict[str, Any], where: str = "config.json") -> Dict[str, Any]:
    """The library's typed, validated reading of a config.json dictionary."""
    if not isinstance(d, dict):
        raise ConfigError(capi.IMP_ERROR_INVALID_MODEL, f"{where}: top level must be an object")
    lib = capi.load()
    return capi.call_json(lib.imp_config_parse, json.dumps(d).encode(), where.encode())


def register_architecture(name: str, config_cls: Type[ModelConfig], plan_fn: Callable[[ModelConfig], Any], *,
                          replace: bool = False) -> None:
    """`plan_fn(config) -> parts.plan.ModelPlan` (or its JSON dictionary)."""
    lib = capi.load()
    if name in _PY_ARCHS or name in known_architectures():
        if not replace:
            raise ValueError(f"architecture '{name}' is already registered")
        unregister_architecture(name)
    holder = {"text": None}

    def plan_callback(_user, config_json):
        try:
            cfg = config_cls.from_json_dict(json.loads(config_json.decode()))
            plan = plan_fn(cfg)
            text = json.dumps(plan.to_json() if hasattr(plan, "to_json") else plan).encode()
            holder["text"] = ctypes.create_string_buffer(text)
            return ctypes.addressof(holder["text"])
        except Exception as e:  # reported through the library's error message
            lib.imp_part_set_error(f"{type(e).__name__}: {e}".encode())
            return None

    cb = capi.PLAN_FN(plan_callback)
    capi.check(lib.imp_register_architecture(name.encode(), cb, None))
    _PY_ARCHS[name] = (config_cls, plan_fn, cb, holder)


def unregister_architecture(name: str) -> None:
    capi.check(capi.load().imp_unregister_architecture(name.encode()))
    _PY_ARCHS.pop(name, None)


def known_architectures():
    return sorted(json.loads(capi.text(capi.load().imp_known_architectures())))


def config_class_of(name: str) -> Type[ModelConfig]:
    if name in _PY_ARCHS:
        return _PY_ARCHS[name][0]
    return _BUILTIN_CONFIGS.get(name, ModelConfig)


def config_from_dict(d: Dict[str, Any], where: str = "config.json") -> ModelConfig:
    archs = d.get("architectures") if isinstance(d, dict) else None
    if not archs or not isinstance(archs, list) or not isinstance(archs[0], str):
        raise ConfigError(capi.IMP_ERROR_INVALID_MODEL, f"{where}: 'architectures' must be a list that names the model class")
    if archs[0] not in known_architectures():
        raise ConfigError(capi.IMP_ERROR_INVALID_MODEL,
                          f"unknown architecture '{archs[0]}'; known: {', '.join(known_architectures()) or '(none)'}")
    return config_class_of(archs[0]).from_json_dict(d, where)


def load_config(model_dir: str) -> ModelConfig:
    path = os.path.join(model_dir, "config.json") if os.path.isdir(model_dir) else model_dir
    if not os.path.exists(path):
        raise ConfigError(capi.IMP_ERROR_FILE_NOT_FOUND, f"no config.json at {path}")
    with open(path) as f:
        try:
            d = json.load(f)
        except json.JSONDecodeError as e:
            raise ConfigError(capi.IMP_ERROR_INVALID_MODEL, f"{path}: not valid JSON: {e}") from None
    if not isinstance(d, dict):
        raise ConfigError(capi.IMP_ERROR_INVALID_MODEL, f"{path}: top level must be an object")
    return config_from_dict(d, path)


def plan_for(config: ModelConfig):
    """The `ModelPlan` (layers, parts, order, tensor names) of a configuration."""
    from ..parts.plan import ModelPlan
    lib = capi.load()
    return ModelPlan.from_json(capi.call_json(lib.imp_plan_for_config, config.to_json().encode()))
