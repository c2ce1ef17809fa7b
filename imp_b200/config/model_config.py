"""Typed model configurations read from an architecture's own config.json keys.

Every size and constant of a model comes from here; no kernel, part or engine
file holds a model size of its own.  The reference keeps one struct for every
family with defaults in the declaration (src/model/model.h:28-76) and never
reads config.json on the safetensors route (src/model/safetensors_loader.cpp:
297-359 infers sizes from tensor shapes); this engine reads config.json and
refuses what it cannot run.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field, fields
from typing import Any, Dict, List, Optional


class ConfigError(ValueError):
    """A config.json that is missing a key, or holds a value the engine cannot run."""


def _require(d: Dict[str, Any], key: str, typ, where: str):
    if key not in d:
        raise ConfigError(f"{where}: missing required key '{key}'")
    v = d[key]
    if typ is float and isinstance(v, int) and not isinstance(v, bool):
        v = float(v)
    if typ is int and isinstance(v, bool):
        raise ConfigError(f"{where}: key '{key}' must be {typ.__name__}, got bool")
    if not isinstance(v, typ):
        raise ConfigError(f"{where}: key '{key}' must be {typ.__name__}, got {type(v).__name__}")
    return v


def _positive(name: str, v, where: str):
    if v <= 0:
        raise ConfigError(f"{where}: '{name}' must be positive, got {v}")
    return v


@dataclass
class ModelConfig:
    """Base of all architecture configurations: the keys every decoder has."""

    architecture: str
    vocab_size: int
    hidden_size: int
    num_hidden_layers: int
    max_position_embeddings: int
    torch_dtype: str = "bfloat16"
    eos_token_id: Optional[int] = None
    bos_token_id: Optional[int] = None
    # Keys of config.json this configuration did not interpret (kept for round trips).
    extra: Dict[str, Any] = field(default_factory=dict)

    # ---- serialisation -------------------------------------------------
    def to_json_dict(self) -> Dict[str, Any]:
        d = {}
        for f in fields(self):
            if f.name in ("architecture", "extra"):
                continue
            v = getattr(self, f.name)
            if v is None:
                continue
            d[f.name] = v
        d["architectures"] = [self.architecture]
        for k, v in self.extra.items():
            d.setdefault(k, v)
        return d

    def save(self, folder: str) -> str:
        os.makedirs(folder, exist_ok=True)
        path = os.path.join(folder, "config.json")
        with open(path, "w") as f:
            json.dump(self.to_json_dict(), f, indent=2, sort_keys=True)
        return path


@dataclass
class Qwen3Config(ModelConfig):
    """The Qwen3 dense decoder (architectures[0] == "Qwen3ForCausalLM").

    Keys follow the HF config.json of this architecture.  The reference reads
    the GGUF twins of the same fields (src/model/gguf_loader.cpp:726-738:
    block_count, embedding_length, head counts, attention.key_length,
    feed_forward_length, rope.freq_base, layer_norm_rms_epsilon; sliding window
    at :821) into src/model/model.h:28-76.
    """

    num_attention_heads: int = 0
    num_key_value_heads: int = 0
    head_dim: int = 0
    intermediate_size: int = 0
    rms_norm_eps: float = 1e-6
    rope_theta: float = 10000.0
    tie_word_embeddings: bool = False
    attention_bias: bool = False
    hidden_act: str = "silu"
    use_sliding_window: bool = False
    sliding_window: Optional[int] = None
    max_window_layers: Optional[int] = None
    layer_types: Optional[List[str]] = None

    KNOWN_KEYS = (
        "architectures", "vocab_size", "hidden_size", "num_hidden_layers",
        "max_position_embeddings", "torch_dtype", "dtype", "eos_token_id", "bos_token_id",
        "num_attention_heads", "num_key_value_heads", "head_dim", "intermediate_size",
        "rms_norm_eps", "rope_theta", "tie_word_embeddings", "attention_bias", "hidden_act",
        "use_sliding_window", "sliding_window", "max_window_layers", "layer_types",
        "rope_scaling", "attention_dropout", "model_type", "initializer_range",
        "use_cache", "transformers_version", "pad_token_id",
    )

    @classmethod
    def from_json_dict(cls, d: Dict[str, Any], where: str = "config.json") -> "Qwen3Config":
        archs = d.get("architectures") or []
        arch = archs[0] if archs else "Qwen3ForCausalLM"
        hidden = _positive("hidden_size", _require(d, "hidden_size", int, where), where)
        heads = _positive("num_attention_heads", _require(d, "num_attention_heads", int, where), where)
        kv_heads = d.get("num_key_value_heads", heads)
        if kv_heads is None:
            kv_heads = heads
        head_dim = d.get("head_dim")
        if head_dim is None:
            if hidden % heads:
                raise ConfigError(f"{where}: no 'head_dim' and hidden_size {hidden} is not a multiple "
                                  f"of num_attention_heads {heads}")
            head_dim = hidden // heads
        dtype = d.get("torch_dtype", d.get("dtype", "bfloat16"))
        eos = d.get("eos_token_id")
        if isinstance(eos, list):
            eos = eos[0] if eos else None
        cfg = cls(
            architecture=arch,
            vocab_size=_positive("vocab_size", _require(d, "vocab_size", int, where), where),
            hidden_size=hidden,
            num_hidden_layers=_positive("num_hidden_layers", _require(d, "num_hidden_layers", int, where), where),
            max_position_embeddings=_positive(
                "max_position_embeddings", int(d.get("max_position_embeddings", 4096)), where),
            torch_dtype=dtype,
            eos_token_id=eos,
            bos_token_id=d.get("bos_token_id"),
            num_attention_heads=heads,
            num_key_value_heads=int(kv_heads),
            head_dim=int(head_dim),
            intermediate_size=_positive("intermediate_size", _require(d, "intermediate_size", int, where), where),
            rms_norm_eps=float(_require(d, "rms_norm_eps", float, where)),
            rope_theta=float(d.get("rope_theta", 10000.0)),
            tie_word_embeddings=bool(d.get("tie_word_embeddings", False)),
            attention_bias=bool(d.get("attention_bias", False)),
            hidden_act=d.get("hidden_act", "silu"),
            use_sliding_window=bool(d.get("use_sliding_window", False)),
            sliding_window=d.get("sliding_window"),
            max_window_layers=d.get("max_window_layers"),
            layer_types=d.get("layer_types"),
            extra={k: v for k, v in d.items() if k not in cls.KNOWN_KEYS},
        )
        if d.get("rope_scaling") not in (None, {}):
            raise ConfigError(f"{where}: rope_scaling {d['rope_scaling']!r} is not supported "
                              "(only the plain rotary encoding)")
        cfg.validate(where)
        return cfg

    def validate(self, where: str = "config") -> None:
        if self.num_key_value_heads <= 0 or self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(f"{where}: num_attention_heads {self.num_attention_heads} must be a positive "
                              f"multiple of num_key_value_heads {self.num_key_value_heads}")
        if self.head_dim <= 0 or self.head_dim % 16:
            raise ConfigError(f"{where}: head_dim {self.head_dim} must be a positive multiple of 16")
        if self.head_dim > 256:
            raise ConfigError(f"{where}: head_dim {self.head_dim} exceeds the kernels' limit of 256")
        if self.attention_bias:
            raise ConfigError(f"{where}: attention_bias=true is not supported for {self.architecture}")
        if self.hidden_act != "silu":
            raise ConfigError(f"{where}: hidden_act '{self.hidden_act}' is not supported (silu only)")
        if self.rms_norm_eps <= 0:
            raise ConfigError(f"{where}: rms_norm_eps must be positive")
        if self.rope_theta <= 0:
            raise ConfigError(f"{where}: rope_theta must be positive")
        if self.torch_dtype not in ("bfloat16", "float32"):
            raise ConfigError(f"{where}: torch_dtype '{self.torch_dtype}' is not supported "
                              "(bfloat16 or float32)")
        if self.layer_types is not None:
            if len(self.layer_types) != self.num_hidden_layers:
                raise ConfigError(f"{where}: layer_types has {len(self.layer_types)} entries for "
                                  f"{self.num_hidden_layers} layers")
            for t in self.layer_types:
                if t not in ("full_attention", "sliding_attention"):
                    raise ConfigError(f"{where}: unknown layer type '{t}'")
        if self.use_sliding_window or (self.layer_types and "sliding_attention" in self.layer_types):
            if not self.sliding_window or self.sliding_window <= 0:
                raise ConfigError(f"{where}: sliding window in use but 'sliding_window' is not a positive size")

    def window_of_layer(self, layer: int) -> int:
        """Window in tokens of `layer` (0 = attends to all earlier tokens).

        A query at position p sees keys j with 0 <= p - j < window, the mask of
        the reference's kernels (src/compute/attention.cu:167; decode:
        src/compute/attention_paged.cu:163-164).
        """
        if self.layer_types is not None:
            return int(self.sliding_window) if self.layer_types[layer] == "sliding_attention" else 0
        if not self.use_sliding_window:
            return 0
        first_window_layer = self.max_window_layers if self.max_window_layers is not None else 0
        return int(self.sliding_window) if layer >= first_window_layer else 0

    def to_json_dict(self) -> Dict[str, Any]:
        d = super().to_json_dict()
        d["model_type"] = "qwen3"
        d.pop("KNOWN_KEYS", None)
        return d
