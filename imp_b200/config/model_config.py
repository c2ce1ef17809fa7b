"""Model configurations as Python objects over the library's typed configurations.

The typed configuration of an architecture (its config.json keys, defaults and
refusals) lives in the library (csrc/host/config.cpp: `Qwen3Config`, which
follows the reference's src/model/model.h:28-76 and gguf_loader.cpp:726-738).
`imp_config_parse` validates a config.json and returns the normalised fields;
the classes here give attribute access to them.
"""
from __future__ import annotations

import json
import os
from typing import Any, Dict, Optional

from ..capi import ConfigError  # noqa: F401  (re-exported)


class ModelConfig:
    """The keys every decoder has; everything else stays reachable through `.extra` and `.raw`."""

    BASE_KEYS = ("architectures", "vocab_size", "hidden_size", "num_hidden_layers", "max_position_embeddings",
                 "torch_dtype", "eos_token_id", "bos_token_id")
    KNOWN_KEYS = BASE_KEYS

    def __init__(self, fields: Dict[str, Any]):
        self.raw: Dict[str, Any] = dict(fields)

    # ---- construction ----------------------------------------------------
    @classmethod
    def from_json_dict(cls, d: Dict[str, Any], where: str = "config.json") -> "ModelConfig":
        from .registry import parse_config_dict
        return cls(parse_config_dict(d, where))

    # ---- fields ----------------------------------------------------------
    @property
    def architecture(self) -> str:
        return self.raw["architectures"][0]

    @property
    def eos_token_ids(self):
        e = self.raw.get("eos_token_id")
        return () if e is None else tuple(e) if isinstance(e, list) else (int(e),)

    @property
    def extra(self) -> Dict[str, Any]:
        return {k: v for k, v in self.raw.items() if k not in self.KNOWN_KEYS}

    def __getattr__(self, name: str):
        raw = self.__dict__.get("raw", {})
        if name in raw:
            return raw[name]
        if name in ("eos_token_id", "bos_token_id", "sliding_window", "max_window_layers", "layer_types"):
            return None
        raise AttributeError(name)

    def __eq__(self, other) -> bool:
        return isinstance(other, ModelConfig) and self.raw == other.raw

    def __repr__(self) -> str:
        return f"{type(self).__name__}({self.raw!r})"

    # ---- serialisation ---------------------------------------------------
    def to_json_dict(self) -> Dict[str, Any]:
        return dict(self.raw)

    def to_json(self) -> str:
        return json.dumps(self.raw)

    def save(self, folder: str) -> str:
        os.makedirs(folder, exist_ok=True)
        path = os.path.join(folder, "config.json")
        with open(path, "w") as f:
            json.dump(self.to_json_dict(), f, indent=2, sort_keys=True)
        return path


class Qwen3Config(ModelConfig):
    """The Qwen3 dense decoder (architectures[0] == "Qwen3ForCausalLM"): num_attention_heads,
    num_key_value_heads, head_dim, intermediate_size, rms_norm_eps, rope_theta, tie_word_embeddings,
    attention_bias, hidden_act, use_sliding_window, sliding_window, max_window_layers, layer_types."""

    KNOWN_KEYS = ModelConfig.BASE_KEYS + (
        "dtype", "num_attention_heads", "num_key_value_heads", "head_dim", "intermediate_size", "rms_norm_eps",
        "rope_theta", "tie_word_embeddings", "attention_bias", "hidden_act", "use_sliding_window", "sliding_window",
        "max_window_layers", "layer_types", "rope_scaling", "attention_dropout", "model_type", "initializer_range",
        "use_cache", "transformers_version", "pad_token_id")

    @classmethod
    def from_json_dict(cls, d: Dict[str, Any], where: str = "config.json") -> "Qwen3Config":
        # validated by the library's Qwen3 configuration, whatever architecture name the folder carries
        from .registry import parse_config_dict
        archs = d.get("architectures")
        probe = dict(d)
        probe["architectures"] = ["Qwen3ForCausalLM"]
        fields = parse_config_dict(probe, where)
        if archs:
            fields["architectures"] = list(archs)
        return cls(fields)

    def window_of_layer(self, layer: int) -> int:
        """Window in tokens of `layer` (0 = attends to all earlier tokens): a query at position p sees
        keys j with 0 <= p - j < window."""
        lt: Optional[list] = self.raw.get("layer_types")
        sw = int(self.raw.get("sliding_window") or 0)
        if lt is not None:
            return sw if lt[layer] == "sliding_attention" else 0
        if not self.raw.get("use_sliding_window"):
            return 0
        first = self.raw.get("max_window_layers")
        return sw if layer >= (first if first is not None else 0) else 0
