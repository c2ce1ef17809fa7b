"""Binds checkpoint tensors to a plan by name, and reports every mismatch at once.

The reference binds by splitting names and treats unknown or missing tensors as
warnings (src/model/weight_map.cpp:152-336; the q/k norm tensors of this family
are dropped on its safetensors route, :295-297).  Here a checkpoint must hold
exactly the tensors the plan expects, with the expected shapes; otherwise one
`WeightError` lists what is missing, what is unexpected and which shapes are
wrong.

Element types on the device:
  compute_dtype bfloat16: floating tensors stored in 16 bits become bfloat16,
      tensors stored in 32 bits stay float32 (the kernels take either), integer
      tables become int32;
  compute_dtype float32: every floating tensor is widened to float32.
"""
from __future__ import annotations

from typing import Dict, List

import torch

from ..parts.plan import ModelPlan, TensorSpec
from .safetensors_io import open_model_files


class WeightError(ValueError):
    """A checkpoint does not match the plan.  `.missing`, `.unexpected`, `.wrong_shape` hold the details."""

    def __init__(self, missing: List[str], unexpected: List[str], wrong_shape: List[str], where: str = ""):
        self.missing, self.unexpected, self.wrong_shape = missing, unexpected, wrong_shape
        lines = [f"checkpoint {where} does not match the model:".replace("  ", " ")]
        if missing:
            lines.append(f"  missing tensors ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            lines.append(f"  unexpected tensors ({len(unexpected)}): " + ", ".join(unexpected))
        if wrong_shape:
            lines.append(f"  wrong shapes ({len(wrong_shape)}): " + "; ".join(wrong_shape))
        super().__init__("\n".join(lines))


def check_names_and_shapes(expected: Dict[str, TensorSpec], found: Dict[str, tuple], where: str = "") -> None:
    missing = sorted(n for n, s in expected.items() if n not in found and not s.optional)
    unexpected = sorted(n for n in found if n not in expected)
    wrong = sorted(f"{n}: expected {list(expected[n].shape)}, found {list(found[n])}"
                   for n in expected if n in found and tuple(found[n]) != tuple(expected[n].shape))
    if missing or unexpected or wrong:
        raise WeightError(missing, unexpected, wrong, where)


def device_dtype(stored: torch.dtype, role: str, compute_dtype: torch.dtype) -> torch.dtype:
    if role == "int_table" or not stored.is_floating_point:
        return torch.int32
    if compute_dtype == torch.float32:
        return torch.float32
    if stored in (torch.float32, torch.float64):
        return torch.float32
    return torch.bfloat16


def load_weights(model_dir: str, plan: ModelPlan, compute_dtype: torch.dtype, device) -> Dict[str, torch.Tensor]:
    """All tensors of the plan, by checkpoint name, on `device`."""
    files = open_model_files(model_dir)
    found_in = {}
    for f in files:
        for name in f.names():
            found_in[name] = f
    expected = plan.expected_tensors()
    check_names_and_shapes(expected, {n: f.info(n)[1] for n, f in found_in.items()}, model_dir)
    out: Dict[str, torch.Tensor] = {}
    for name, spec in expected.items():
        if name not in found_in:
            continue  # optional and absent
        src = found_in[name].tensor(name)
        out[name] = place_tensor(src, spec.role, compute_dtype, device)
    for f in files:
        f.close()
    return out


def place_tensor(src: torch.Tensor, role: str, compute_dtype: torch.dtype, device) -> torch.Tensor:
    """Copy one checkpoint tensor to the device in the element type the engine keeps it in."""
    dt = device_dtype(src.dtype, role, compute_dtype)
    dev = torch.device(device)
    if dev.type == "cpu":
        return src.to(dt).contiguous().clone() if src.dtype == dt else src.to(dt).contiguous()
    # Convert on the device: the host copy stays in its stored type (no widened temporary on the host).
    t = src.to(dev, non_blocking=False)
    return t.to(dt).contiguous() if t.dtype != dt else t.contiguous()
