"""The data that describes a model: which parts, with which sizes, in which order.

A `ModelPlan` is what an architecture's plan function makes out of its typed
configuration.  It is pure data: part kinds are names resolved through
imp_b200/parts/registry.py, sizes and constants are parameters, tensor names are
the checkpoint's own, and the order in which layers run is a list (which may
name a layer twice).  A layer may read another layer's cache (`cache_from`).
The reference has no such description: its forward pass is one hard-coded
function that switches on tensor presence (src/graph/executor_forward.cu:
2701-3140, layer kinds at src/graph/executor_workspace.cu:2314-2330).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple


@dataclass
class PartSpec:
    """One part: its kind, its parameters, and the checkpoint name of each of its tensors."""

    kind: str
    params: Dict[str, Any] = field(default_factory=dict)
    tensors: Dict[str, str] = field(default_factory=dict)  # local name -> checkpoint tensor name

    def key(self) -> str:
        return repr((self.kind, sorted((k, repr(v)) for k, v in self.params.items()),
                     sorted(self.tensors.items())))


@dataclass
class LayerSpec:
    """One layer: a mixer and a feed-forward with their norms, arranged by `block`."""

    mixer: PartSpec
    feed_forward: PartSpec
    mixer_norm: PartSpec
    ffn_norm: PartSpec
    block: str = "prenorm"
    cache_from: Optional[int] = None  # index of the layer whose cache this layer reads (it writes none)


@dataclass
class TensorSpec:
    """What a part expects of one checkpoint tensor."""

    shape: Tuple[int, ...]
    role: str = "matrix"      # "matrix" | "norm" | "int_table" | "vector"
    init: str = "normal"      # random-weights rule: "normal" | "one_plus_normal" | "zeros" | "arange_mod"
    optional: bool = False


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

    def run_order(self) -> List[int]:
        order = list(range(len(self.layers))) if self.order is None else list(self.order)
        for i in order:
            if not 0 <= i < len(self.layers):
                raise ValueError(f"run order names layer {i}, but the plan has {len(self.layers)} layers")
        return order

    def part_specs(self):
        """(category, spec) for every part of the plan, in a fixed order."""
        yield "embedding", self.embedding
        for layer in self.layers:
            yield "norm", layer.mixer_norm
            yield "mixer", layer.mixer
            yield "norm", layer.ffn_norm
            yield "feed_forward", layer.feed_forward
        yield "norm", self.final_norm
        yield "head", self.head

    def expected_tensors(self) -> Dict[str, TensorSpec]:
        """Checkpoint tensor name -> what is expected of it, over all parts.

        Two parts may name the same tensor (a tied output head); their
        expectations must then agree on the shape.
        """
        from .registry import part_class

        out: Dict[str, TensorSpec] = {}
        for category, spec in self.part_specs():
            cls = part_class(category, spec.kind)
            for local, ts in cls.tensor_specs(spec.params).items():
                if local not in spec.tensors:
                    if ts.optional:
                        continue
                    raise ValueError(f"plan error: part '{spec.kind}' needs a checkpoint name for its tensor '{local}'")
                name = spec.tensors[local]
                if name in out:
                    if tuple(out[name].shape) != tuple(ts.shape):
                        raise ValueError(f"plan error: tensor '{name}' is used with shapes "
                                         f"{out[name].shape} and {ts.shape}")
                    continue
                out[name] = ts
        return out
