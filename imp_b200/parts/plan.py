"""The data that describes a model, as Python objects over the library's plan JSON.

A `ModelPlan` is what an architecture's plan function makes out of its
configuration: part kinds (names resolved through the library's part
registry), sizes and constants as parameters, the checkpoint's own tensor
names, layers as a block kind with named part slots, and the order in which
layers run as a list (which may name a layer twice).  A layer may read another
layer's cache (`cache_from`).  The library's own plans (csrc/host/config.cpp
`qwen3_plan`) come back from `plan_for` in this form, so a plan function
written in Python can start from one and change it.  The JSON layout is given
in include/imp_b200/imp_parts.h.
"""
from __future__ import annotations

import json
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple


@dataclass
class PartSpec:
    """One part: its kind, its parameters, and the checkpoint name of each of its tensors."""

    kind: str
    params: Dict[str, Any] = field(default_factory=dict)
    tensors: Dict[str, str] = field(default_factory=dict)  # local name -> checkpoint tensor name

    def to_json(self) -> Dict[str, Any]:
        params = {k: (v.to_json() if isinstance(v, PartSpec) else v) for k, v in self.params.items()}
        return {"kind": self.kind, "params": params, "tensors": dict(self.tensors)}

    @classmethod
    def from_json(cls, j: Dict[str, Any]) -> "PartSpec":
        return cls(j["kind"], dict(j.get("params") or {}), dict(j.get("tensors") or {}))


class LayerSpec:
    """One layer: a block kind (`block`, `block_params`) and the parts in the slots that block declares
    (`parts`: slot name -> PartSpec).  The usual slots (mixer, feed_forward, mixer_norm, ffn_norm) can be
    named as keyword arguments and attributes.  `cache_from`: index of the layer whose cache this layer's
    mixer reads (it writes none)."""

    def __init__(self, block: str = "prenorm", parts: Optional[Dict[str, PartSpec]] = None,
                 block_params: Optional[Dict[str, Any]] = None, cache_from: Optional[int] = None, **slots: PartSpec):
        self.block = block
        self.parts = dict(parts or {})
        self.parts.update(slots)
        self.block_params = dict(block_params or {})
        self.cache_from = cache_from

    def __getattr__(self, name: str):
        parts = self.__dict__.get("parts")
        if parts is not None and name in parts:
            return parts[name]
        raise AttributeError(name)

    def __setattr__(self, name: str, value) -> None:
        if name in ("block", "parts", "block_params", "cache_from"):
            object.__setattr__(self, name, value)
        else:
            self.parts[name] = value

    def to_json(self) -> Dict[str, Any]:
        return {"block": self.block, "block_params": self.block_params,
                "parts": {k: v.to_json() for k, v in self.parts.items()}, "cache_from": self.cache_from}

    @classmethod
    def from_json(cls, j: Dict[str, Any]) -> "LayerSpec":
        return cls(j.get("block", "prenorm"), {k: PartSpec.from_json(v) for k, v in j["parts"].items()},
                   j.get("block_params") or {}, j.get("cache_from"))


@dataclass
class TensorSpec:
    """What a part expects of one checkpoint tensor."""

    shape: Tuple[int, ...]
    role: str = "matrix"      # "matrix" | "norm" | "int_table" | "vector"
    init: str = "normal"      # random-weights rule: "normal" | "one_plus_normal" | "zeros" | "arange_mod"
    optional: bool = False

    def to_json(self) -> Dict[str, Any]:
        return {"shape": list(self.shape), "role": self.role, "init": self.init, "optional": self.optional}

    @classmethod
    def from_json(cls, j: Dict[str, Any]) -> "TensorSpec":
        return cls(tuple(j["shape"]), j.get("role", "matrix"), j.get("init", "normal"), bool(j.get("optional", False)))


@dataclass
class ModelPlan:
    architecture: str
    hidden_size: int
    vocab_size: int
    embedding: PartSpec
    layers: List[LayerSpec]
    final_norm: PartSpec
    head: PartSpec
    order: Optional[List[int]] = None  # run order of layer indices; None = 0..L-1
    max_positions: int = 4096
    ignored_tensors: List[str] = field(default_factory=list)

    def run_order(self) -> List[int]:
        order = list(range(len(self.layers))) if self.order is None else list(self.order)
        for i in order:
            if not 0 <= i < len(self.layers):
                raise ValueError(f"run order names layer {i}, but the plan has {len(self.layers)} layers")
        return order

    def to_json(self) -> Dict[str, Any]:
        return {"architecture": self.architecture, "hidden_size": self.hidden_size, "vocab_size": self.vocab_size,
                "max_positions": self.max_positions, "embedding": self.embedding.to_json(),
                "layers": [l.to_json() for l in self.layers], "final_norm": self.final_norm.to_json(),
                "head": self.head.to_json(), "order": None if self.order is None else list(self.order),
                "ignored_tensors": list(self.ignored_tensors)}

    @classmethod
    def from_json(cls, j: Dict[str, Any]) -> "ModelPlan":
        return cls(j.get("architecture", ""), j["hidden_size"], j["vocab_size"], PartSpec.from_json(j["embedding"]),
                   [LayerSpec.from_json(l) for l in j["layers"]], PartSpec.from_json(j["final_norm"]),
                   PartSpec.from_json(j["head"]), j.get("order"), j.get("max_positions", 4096),
                   list(j.get("ignored_tensors") or []))

    def expected_tensors(self) -> Dict[str, TensorSpec]:
        """Checkpoint tensor name -> what is expected of it, over all parts (asked of the library)."""
        from .. import capi
        j = capi.call_json(capi.load().imp_plan_expected_tensors, json.dumps(self.to_json()).encode())
        return {name: TensorSpec.from_json(spec) for name, spec in j.items()}
