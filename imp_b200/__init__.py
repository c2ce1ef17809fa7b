"""imp_b200: a small inference engine for one B200 GPU and the Qwen3 dense decoder.

The engine is a C++/CUDA library with a C API (include/imp_b200/imp.h); this package is the
thin Python entry point over it.

Public names:
    Engine, Model, EngineConfig, GenerateParams   the entry point (imp_b200/engine/engine.py)
    StepEntry                                     one request's next tokens for `Engine.step_tokens`
    load_config, config_from_dict, plan_for       configuration and the plan of a model
    register_architecture, register_part          architectures and part kinds added from Python
    write_model_folder                            a model folder with random weights from a configuration
"""
from .capi import ConfigError, ImpError, KernelError, OutOfPages, WeightError
from .config.engine_config import EngineConfig
from .config.model_config import ModelConfig, Qwen3Config
from .config.registry import (config_from_dict, load_config, plan_for, register_architecture,
                              unregister_architecture)
from .engine.engine import Engine, GenerateParams, Model, StepEntry
from .parts.registry import register_part, unregister_part
from .weights.random_init import write_model_folder

__version__ = "0.2.0"

__all__ = ["Engine", "Model", "EngineConfig", "GenerateParams", "StepEntry", "ConfigError", "ImpError", "KernelError",
           "OutOfPages", "WeightError", "ModelConfig", "Qwen3Config", "config_from_dict", "load_config", "plan_for",
           "register_architecture", "unregister_architecture", "register_part", "unregister_part", "write_model_folder"]
