"""From a model folder (or a configuration and a seed) to a model ready to step."""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from ..cache.manager import CacheManager
from ..config.model_config import ModelConfig
from ..config.registry import load_config, plan_for
from ..ops import kernels as K
from ..ops import library
from ..parts.base import Runtime
from ..weights.loader import check_names_and_shapes, load_weights, place_tensor
from ..weights.random_init import random_tensor
from .model import DecoderModel

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32}


def parse_dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        if name not in (torch.bfloat16, torch.float32):
            raise ValueError(f"compute dtype must be bfloat16 or float32, got {name}")
        return name
    try:
        return _DTYPES[str(name).lower()]
    except KeyError:
        raise ValueError(f"compute dtype must be bfloat16 or float32, got {name!r}") from None


def make_runtime(dtype, device, max_positions: int) -> Runtime:
    library.require_device()
    device = torch.device(device)
    return Runtime(dtype=parse_dtype(dtype), device=device, status=K.new_status(device), max_positions=max_positions)


def load_model(model_dir: str, dtype="bfloat16", device="cuda:0") -> Tuple[ModelConfig, DecoderModel]:
    """Read config.json, pick the architecture, load model.safetensors, build the parts."""
    config = load_config(model_dir)
    plan = plan_for(config)
    rt = make_runtime(dtype, device, plan.max_positions)
    with torch.cuda.device(rt.device):
        tensors = load_weights(model_dir, plan, rt.dtype, rt.device)
        return config, DecoderModel(plan, tensors, rt)


def model_from_tensors(config: ModelConfig, tensors: Dict[str, torch.Tensor], dtype="bfloat16",
                       device="cuda:0") -> DecoderModel:
    """Build a model from tensors by checkpoint name (host or device); names and shapes are checked."""
    plan = plan_for(config)
    rt = make_runtime(dtype, device, plan.max_positions)
    expected = plan.expected_tensors()
    check_names_and_shapes(expected, {n: tuple(t.shape) for n, t in tensors.items()}, "(in memory)")
    with torch.cuda.device(rt.device):
        placed = {n: place_tensor(t, expected[n].role, rt.dtype, rt.device) for n, t in tensors.items()}
        return DecoderModel(plan, placed, rt)


def random_model(config: ModelConfig, seed: int = 0, std: float = 0.02, norm_std: float = 0.01,
                 dtype="bfloat16", device="cuda:0", store_dtype: Optional[torch.dtype] = None) -> DecoderModel:
    """A model with random weights made on the device, tensor by tensor (nothing touches the disk).

    Values are a function of (seed, tensor name) for a given device type; a folder written by
    `weights.random_init.write_model_folder` uses the host generator and holds other values.
    """
    plan = plan_for(config)
    rt = make_runtime(dtype, device, plan.max_positions)
    store = store_dtype or getattr(torch, config.torch_dtype)
    with torch.cuda.device(rt.device):
        placed = {}
        for name, spec in plan.expected_tensors().items():
            t = random_tensor(name, spec, seed, std, norm_std, store, rt.device)
            placed[name] = place_tensor(t, spec.role, rt.dtype, rt.device)
        return DecoderModel(plan, placed, rt)


def make_cache(model: DecoderModel, page_size: int, num_pages: int, num_slots: int) -> CacheManager:
    """A cache manager with device storage for `model` (groups follow the model's run positions)."""
    cache = CacheManager(model.cache_specs, page_size, num_pages, num_slots)
    with torch.cuda.device(model.rt.device):
        cache.allocate_storage(model.rt.dtype, model.rt.device)
    return cache
