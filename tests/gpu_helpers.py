"""Helpers for GPU tests that drive single parts: a batch context from the engine's own step
function, without a model."""
import torch

from imp_b200.cache.manager import CacheManager
from imp_b200.engine.step import StepEntry, Stepper
from imp_b200.ops import kernels as K
from imp_b200.parts.base import LayerCache, Runtime

DEV = "cuda:0"


class NoModel:
    """Stands where the step function expects a model; only the batch arrays are wanted."""

    def __init__(self, vocab_size=1 << 20):
        self.vocab_size = vocab_size

    def attach_cache(self, cache):
        pass


def runtime(dtype, max_positions=512):
    from imp_b200.ops import library
    library.require_device()
    return Runtime(dtype=dtype, device=torch.device(DEV), status=K.new_status(DEV), max_positions=max_positions)


def part_stepper(cache_specs, rt, page_size=4, num_pages=64, slots=4, max_tokens=256, max_seq_len=256):
    cache = CacheManager(cache_specs, page_size, num_pages, slots)
    cache.allocate_storage(rt.dtype, rt.device)
    return Stepper(NoModel(), cache, rt, max_tokens, slots, max_seq_len), cache


def layer_cache(cache, ctx, position=0, writes=True):
    kind, storage = cache.layer_storage(position)
    if kind == "paged":
        g = cache.layer_ref[position].group
        return LayerCache("paged", kv=storage, block_table=ctx.block_tables[g], writes=writes,
                          page_size=cache.page_size, group=g)
    return LayerCache("state", state=storage, writes=writes, group=cache.layer_ref[position].group)


def dummy_entries(lengths, rid_prefix="s"):
    return [StepEntry(f"{rid_prefix}{i}", [1] * n, []) for i, n in enumerate(lengths)]
