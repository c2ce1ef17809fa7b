"""Interfaces of the parts a model is put together from.

A part is built from (params, tensors, runtime): `params` are its sizes and
constants (from the plan, never from a model class), `tensors` its weights by
local name, `runtime` the precision, the device and the status word.  No part
knows which model it is in.

Categories and what each must provide:

  norm          add_norm(h, branch, rows=None) -> normalised activations;
                h is the 32-bit residual stream, `branch` (or None) is added
                into it first; with `rows` only those rows are produced and h
                is left as it is.
  position      rotary_tables() -> (cos, sin, rotary_dim) or None;
                apply(q, k, ctx) for encodings the fused kernel cannot express.
  mixer         cache_spec(params) (classmethod) -> PagedKVSpec | StateSpec | None;
                forward(x, ctx, cache) -> [T, hidden] branch output.
  feed_forward  forward(x, ctx) -> [T, hidden] branch output.
  block         forward(h, pending, ctx, cache) -> (h, pending): the arrangement
                of one layer's norms, mixer and feed-forward around the stream.
  embedding     forward(token_ids, ctx) -> [T, hidden] float32 stream.
  head          forward(x_rows) -> [R, vocab] float32 logits.

Every part class also provides `tensor_specs(params)` (classmethod): the
checkpoint tensors it needs, by local name, with shapes.

Unsummed branch outputs.  A matrix product of few rows is cut over the
contraction and leaves partial results that someone has to add
(ops.kernels.SplitSum).  A norm that can add them while it reads the branch
sets `takes_split_sum = True`; a mixer or feed-forward whose `defer_out` has
been set to True by whoever arranges it may then return a SplitSum instead of
a tensor.  Both default to False, so a part that knows nothing of this never
meets one.  A block says through `takes_split_sum` whether the `pending` it is
given may be one, and is told through `defer_pending` whether the `pending`
it returns may be one.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, Optional

import torch

from .plan import TensorSpec


@dataclass
class Runtime:
    """What every part is built with."""

    dtype: torch.dtype            # activation/cache element type: torch.bfloat16 or torch.float32
    device: torch.device
    status: Optional[torch.Tensor] = None   # device status word (int32[1])
    max_positions: int = 4096
    shared: Dict[Any, Any] = field(default_factory=dict)   # parts without tensors, shared between equal specs

    @property
    def is_float32(self) -> bool:
        return self.dtype == torch.float32

    def empty(self, shape, dtype=None) -> torch.Tensor:
        return torch.empty(shape, dtype=dtype or self.dtype, device=self.device)


class Part:
    category = "part"
    takes_split_sum = False   # norm: add_norm accepts an unsummed branch
    defer_out = False         # mixer, feed_forward: forward may return an unsummed branch

    def __init__(self, params: Dict[str, Any], tensors: Dict[str, torch.Tensor], rt: Runtime):
        self.params = params
        self.tensors = tensors
        self.rt = rt

    @classmethod
    def tensor_specs(cls, params: Dict[str, Any]) -> Dict[str, TensorSpec]:
        return {}


class Norm(Part):
    category = "norm"

    def add_norm(self, h: torch.Tensor, branch: Optional[torch.Tensor],
                 rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        raise NotImplementedError


class PositionEncoding(Part):
    category = "position"

    def rotary_tables(self):
        """(cos[max_pos, rot/2], sin[...], rot_dim) for rotary encodings, else None."""
        return None

    def apply(self, q: torch.Tensor, k: torch.Tensor, ctx) -> None:
        """Encode positions into q [T, Hq, Dh] and k [T, Hkv, Dh] in place (unfused path)."""
        raise NotImplementedError


class Mixer(Part):
    category = "mixer"

    @classmethod
    def cache_spec(cls, params: Dict[str, Any]):
        return None

    def forward(self, x: torch.Tensor, ctx, cache) -> torch.Tensor:
        raise NotImplementedError


class FeedForward(Part):
    category = "feed_forward"

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        raise NotImplementedError


class Embedding(Part):
    category = "embedding"

    def forward(self, token_ids: torch.Tensor, ctx) -> torch.Tensor:
        raise NotImplementedError


class Head(Part):
    category = "head"

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError


@dataclass
class LayerCache:
    """What a mixer gets of the cache for one step.

    kind "paged": `kv` is [2, pages, kv_heads, page_size, head_dim] (0 = keys, 1 = values),
    `block_table` [B, max_pages] int32 rows in batch order, `writes` tells whether this layer
    owns the cache (False when it reads another layer's).
    kind "state": `state` is [slots, *shape]; the request's slot ids are ctx.state_slots, and
    ctx.fresh marks requests whose state starts at zero in this step.
    """

    kind: str
    kv: Optional[torch.Tensor] = None
    block_table: Optional[torch.Tensor] = None
    state: Optional[torch.Tensor] = None
    writes: bool = True
    page_size: int = 0
    group: int = 0   # index of the cache group (block tables and state storage are per group)


class Block:
    """Arrangement of one layer.  Built from the layer's already built parts."""

    category = "block"
    takes_split_sum = False   # the pending it is given may be an unsummed branch
    defer_pending = False     # set by the model: the pending it returns may be an unsummed branch

    def __init__(self, mixer: Mixer, feed_forward: FeedForward, mixer_norm: Norm, ffn_norm: Norm, rt: Runtime):
        self.mixer = mixer
        self.feed_forward = feed_forward
        self.mixer_norm = mixer_norm
        self.ffn_norm = ffn_norm
        self.rt = rt

    def forward(self, h: torch.Tensor, pending: Optional[torch.Tensor], ctx, cache: Optional[LayerCache]):
        raise NotImplementedError
