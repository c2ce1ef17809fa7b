"""A model assembled from a plan: embedding, blocks in their run order, final norm, head.

`DecoderModel.forward(ctx)` is the whole forward pass of one step over the
batch `ctx` describes; it runs only the tokens it is given, reads and writes
the cache through the per-position `LayerCache` objects, and returns 32-bit
logits for the rows that were asked for.  It is the same function for whole
prompts, portions, single decode tokens and any mix of them (the reference has
separate prefill and decode paths and no mixed batch:
src/graph/executor_forward.cu:568-701).

Cache ownership follows the run order, not the layer list: every position of
the run order whose layer owns a cache gets a cache of its own (a layer named
twice must not overwrite its first pass's keys), and a layer with `cache_from`
reads the cache of the latest earlier position that ran that other layer.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..cache.manager import CacheManager
from ..parts.base import LayerCache, Runtime
from ..parts.builtin import build_part
from ..parts.plan import ModelPlan
from ..parts.registry import part_class


class DecoderModel:
    def __init__(self, plan: ModelPlan, tensors: Dict[str, torch.Tensor], rt: Runtime):
        self.plan = plan
        self.rt = rt
        self.hidden_size = plan.hidden_size
        self.vocab_size = plan.vocab_size

        def take(spec):
            return {local: tensors[name] for local, name in spec.tensors.items() if name in tensors}

        self.embedding = build_part("embedding", plan.embedding, take(plan.embedding), rt)
        self.blocks = []
        for layer in plan.layers:
            mixer = build_part("mixer", layer.mixer, take(layer.mixer), rt)
            ffn = build_part("feed_forward", layer.feed_forward, take(layer.feed_forward), rt)
            n1 = build_part("norm", layer.mixer_norm, take(layer.mixer_norm), rt)
            n2 = build_part("norm", layer.ffn_norm, take(layer.ffn_norm), rt)
            self.blocks.append(part_class("block", layer.block)(mixer, ffn, n1, n2, rt))
        self.final_norm = build_part("norm", plan.final_norm, take(plan.final_norm), rt)
        self.head = build_part("head", plan.head, take(plan.head), rt)

        self.order: List[int] = plan.run_order()
        # A block may hand on an unsummed branch only if whoever normalises the stream after it, at every place
        # it has in the run order, adds the parts itself.
        after_ok = {i: True for i in range(len(self.blocks))}
        for j, i in enumerate(self.order):
            nxt = self.blocks[self.order[j + 1]] if j + 1 < len(self.order) else self.final_norm
            after_ok[i] = after_ok[i] and bool(nxt.takes_split_sum)
        for i, blk in enumerate(self.blocks):
            blk.defer_pending = after_ok[i]
        # Cache needs per run position, and which position's cache each position uses.
        self.cache_specs: List[Optional[object]] = []
        self.cache_position: List[int] = []
        last_position_of_layer: Dict[int, int] = {}
        for j, i in enumerate(self.order):
            layer = plan.layers[i]
            if layer.cache_from is None:
                cls = part_class("mixer", layer.mixer.kind)
                self.cache_specs.append(cls.cache_spec(layer.mixer.params))
                self.cache_position.append(j)
            else:
                if layer.cache_from not in last_position_of_layer:
                    raise ValueError(f"layer {i} reads the cache of layer {layer.cache_from}, "
                                     "which has not run before it in the run order")
                self.cache_specs.append(None)
                self.cache_position.append(last_position_of_layer[layer.cache_from])
            if layer.cache_from is None:
                last_position_of_layer[i] = j
        self.layer_caches: List[Optional[LayerCache]] = [None] * len(self.order)
        self.cache: Optional[CacheManager] = None

    # ------------------------------------------------------------------ cache
    def attach_cache(self, cache: CacheManager) -> None:
        """Bind the cache manager's storage to the run positions."""
        self.cache = cache
        for j in range(len(self.order)):
            src = self.cache_position[j]
            kind, storage = cache.layer_storage(src)
            if kind is None:
                self.layer_caches[j] = None
            elif kind == "paged":
                self.layer_caches[j] = LayerCache("paged", kv=storage, writes=(src == j),
                                                  page_size=cache.page_size)
                self.layer_caches[j].group = cache.layer_ref[src].group
            else:
                self.layer_caches[j] = LayerCache("state", state=storage, writes=(src == j))
                self.layer_caches[j].group = cache.layer_ref[src].group

    # ---------------------------------------------------------------- forward
    def forward(self, ctx) -> torch.Tensor:
        """Run the batch; returns float32 logits [len(ctx.logit_rows), vocab]."""
        for lc in self.layer_caches:
            if lc is not None and lc.kind == "paged":
                lc.block_table = ctx.block_tables[lc.group]
        h = self.embedding.forward(ctx.token_ids, ctx)
        pending = None
        for j, i in enumerate(self.order):
            h, pending = self.blocks[i].forward(h, pending, ctx, self.layer_caches[j])
        if ctx.n_rows == 0:
            return torch.empty((0, self.vocab_size), dtype=torch.float32, device=self.rt.device)
        x = self.final_norm.add_norm(h, pending, rows=ctx.logit_rows)
        return self.head.forward(x)
