"""imp_b200: a small inference engine for one B200 GPU and the Qwen3 dense decoder.

Public names:
    Engine, EngineConfig, GenerateParams   the entry point (imp_b200/engine/engine.py)
    StepEntry                              one request's next tokens for `Engine.step_tokens`
    load_config, register_architecture     configuration and the architecture registry
    register_part                          new part kinds (mixer, feed_forward, norm, position, ...)
    write_model_folder                     a model folder with random weights from a configuration
"""
from .config.engine_config import EngineConfig
from .config.model_config import ConfigError, ModelConfig, Qwen3Config
from .config.registry import config_from_dict, load_config, plan_for, register_architecture
from .parts.registry import register_part
from .weights.random_init import write_model_folder

__version__ = "0.1.0"

__all__ = ["Engine", "EngineConfig", "GenerateParams", "StepEntry", "ConfigError", "ModelConfig", "Qwen3Config",
           "config_from_dict", "load_config", "plan_for", "register_architecture", "register_part",
           "write_model_folder"]


def __getattr__(name):
    # The engine pulls in torch.cuda-facing modules; load it on first use.
    if name in ("Engine", "GenerateParams"):
        from .engine import engine as _e
        return getattr(_e, name)
    if name == "StepEntry":
        from .engine.step import StepEntry
        return StepEntry
    raise AttributeError(name)
