"""Random weights by tensor name from a configuration and a seed.

Each tensor has a generator of its own, seeded from (seed, tensor name), so a
tensor's values do not depend on which other tensors exist or in which order
they are made.  Matrices are N(0, std); norm weights are 1 + N(0, norm_std);
integer tables are index mod 2^15.  `write_model_folder` stores the result as a
model folder (config.json + model.safetensors) that loads like any checkpoint.
The reference fills test and bench models from one std::mt19937(42) stream,
uniform in +-0.01 with norm weights 1.0 (tools/imp-bench/bench_e2e.cpp:43-120).
"""
from __future__ import annotations

import hashlib
import os
from typing import Dict, Optional

import torch

from ..config.model_config import ModelConfig
from ..config.registry import plan_for
from ..parts.plan import ModelPlan, TensorSpec
from .safetensors_io import save_safetensors


def tensor_seed(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{int(seed)}:{name}".encode()).digest()
    return int.from_bytes(h[:8], "little") & 0x7FFFFFFFFFFFFFFF


def random_tensor(name: str, spec: TensorSpec, seed: int, std: float, norm_std: float,
                  dtype: torch.dtype, device="cpu") -> torch.Tensor:
    dev = torch.device(device)
    g = torch.Generator(device=dev)
    g.manual_seed(tensor_seed(seed, name))
    if spec.role == "int_table" or spec.init == "arange_mod":
        n = 1
        for s in spec.shape:
            n *= s
        return (torch.arange(n, device=dev, dtype=torch.int64) % 32768).to(torch.int32).reshape(spec.shape)
    if spec.init == "zeros":
        return torch.zeros(spec.shape, dtype=dtype, device=dev)
    x = torch.randn(spec.shape, generator=g, dtype=torch.float32, device=dev)
    if spec.init == "one_plus_normal":
        x.mul_(norm_std).add_(1.0)
    else:
        x.mul_(std)
    return x.to(dtype)


def random_tensors(plan: ModelPlan, seed: int = 0, std: float = 0.02, norm_std: float = 0.01,
                   dtype: torch.dtype = torch.bfloat16, device="cpu") -> Dict[str, torch.Tensor]:
    """name -> tensor for every tensor of the plan, stored as `dtype`."""
    return {name: random_tensor(name, spec, seed, std, norm_std, dtype, device)
            for name, spec in plan.expected_tensors().items()}


def write_model_folder(folder: str, config: ModelConfig, seed: int = 0, std: float = 0.02,
                       norm_std: float = 0.01, dtype: Optional[torch.dtype] = None) -> str:
    """Write config.json and model.safetensors with random weights; returns the folder."""
    if dtype is None:
        dtype = getattr(torch, config.torch_dtype)
    os.makedirs(folder, exist_ok=True)
    config.save(folder)
    tensors = random_tensors(plan_for(config), seed, std, norm_std, dtype, "cpu")
    save_safetensors(os.path.join(folder, "model.safetensors"), tensors,
                     {"format": "pt", "seed": str(seed), "std": str(std)})
    return folder
