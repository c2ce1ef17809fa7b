"""The Qwen3 dense decoder's plan, as a starting point for plan functions written in Python.

The plan itself is made by the library (csrc/host/config.cpp `qwen3_plan`: pre-norm blocks of
grouped-query attention with per-head RMSNorm on q and k before the rotary encoding, a SwiGLU
feed-forward, final RMSNorm, tied or untied head; the reference's forward pass for this family is
src/graph/executor_forward.cu:2701-3140).  `qwen3_plan(cfg)` returns it for any configuration that
carries this family's keys, whatever architecture name it has, so that another architecture can
take it and swap parts, share caches or change the run order.
"""
from __future__ import annotations

from ..config.model_config import ModelConfig, Qwen3Config
from ..config.registry import plan_for
from ..parts.plan import ModelPlan


def qwen3_plan(cfg: ModelConfig) -> ModelPlan:
    fields = dict(cfg.raw)
    fields["architectures"] = ["Qwen3ForCausalLM"]
    plan = plan_for(Qwen3Config(fields))
    plan.architecture = cfg.architecture
    return plan
