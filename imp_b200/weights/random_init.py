"""Random weights by tensor name from a configuration and a seed, written as a model folder.

Each tensor is a function of (seed, tensor name) alone, so its values do not
depend on which other tensors exist or in which order they are made.  Matrices
are N(0, std); norm weights are 1 + N(0, norm_std); integer tables are index
mod 2^15.  The generator and the safetensors writer are the library's
(csrc/host/weights.cpp); the folder (config.json + model.safetensors) loads
like any checkpoint.  The reference fills test and bench models from one
std::mt19937(42) stream, uniform in +-0.01 with norm weights 1.0
(tools/imp-bench/bench_e2e.cpp:43-120).
"""
from __future__ import annotations

from typing import Optional

from .. import capi
from ..config.model_config import ModelConfig


def write_model_folder(folder: str, config: ModelConfig, seed: int = 0, std: float = 0.02, norm_std: float = 0.01,
                       dtype: Optional[str] = None) -> str:
    """Write config.json and model.safetensors with random weights; returns the folder.
    `dtype`: "bfloat16" or "float32" (default: the configuration's torch_dtype)."""
    if dtype is not None and not isinstance(dtype, str):
        dtype = str(dtype).replace("torch.", "")
    lib = capi.load()
    capi.model_error(lib.imp_model_write_random(config.to_json().encode(), folder.encode(), int(seed), float(std),
                                                float(norm_std), dtype.encode() if dtype else None))
    return folder
