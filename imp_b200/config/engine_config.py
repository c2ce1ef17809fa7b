"""Engine settings, with the reference's field names where it has them.

`device_id`, `max_batch_size`, `max_seq_len`, `kv_cache_max_blocks`,
`compute_dtype`, `prefill_chunk_size`, `enable_cuda_graphs` come from
include/imp/config.h:11-81 (defaults: src/api/imp_api.cpp:35-72);
`kv_block_size` from src/runtime/engine.h:59.  `max_batch_tokens` (the token
budget of one step) and `lookahead` are this engine's own.  The dataclass
mirrors the C API's `ImpConfig` (include/imp_b200/imp.h).
"""
from __future__ import annotations

from dataclasses import dataclass

from .. import capi


@dataclass
class EngineConfig:
    device_id: int = 0
    max_batch_size: int = 32          # requests decoded together (reference default 32)
    max_seq_len: int = 4096           # longest context of one request (reference default 4096)
    kv_cache_max_blocks: int = 0      # pages per cache group; 0 = from kv_cache_tokens / memory
    kv_cache_tokens: int = 0          # pool size in tokens when kv_cache_max_blocks == 0
    kv_block_size: int = 16           # tokens per page
    prefill_chunk_size: int = 0       # longest portion of one prompt in a step; 0 = no cut
    max_batch_tokens: int = 2048      # token budget of one step (decodes + prompt portions)
    compute_dtype: str = "bfloat16"   # "bfloat16" or "float32"
    enable_cuda_graphs: bool = True   # capture decode-only steps
    gpu_memory_fraction: float = 0.8  # of free memory to the cache when nothing else sizes it
    state_slots: int = 0              # fixed-size state slots; 0 = max_batch_size
    lookahead: bool = True            # launch the next decode step before reading the last one's tokens

    def validate(self) -> None:
        if self.compute_dtype not in ("bfloat16", "float32"):
            raise ValueError(f"compute_dtype must be 'bfloat16' or 'float32', got {self.compute_dtype!r}")
        for name in ("max_batch_size", "max_seq_len", "kv_block_size", "max_batch_tokens"):
            if getattr(self, name) <= 0:
                raise ValueError(f"{name} must be positive")
        if self.prefill_chunk_size < 0:
            raise ValueError("prefill_chunk_size must be >= 0")
        if self.max_batch_tokens < self.max_batch_size:
            raise ValueError("max_batch_tokens must be at least max_batch_size (one token per decoding request)")

    def to_c(self) -> "capi.ImpConfig":
        self.validate()
        c = capi.load().imp_config_default()
        c.device_id = self.device_id
        c.kv_cache_max_blocks = self.kv_cache_max_blocks
        c.kv_cache_tokens = self.kv_cache_tokens
        c.kv_block_size = self.kv_block_size
        c.max_batch_size = self.max_batch_size
        c.max_seq_len = self.max_seq_len
        c.max_batch_tokens = self.max_batch_tokens
        c.prefill_chunk_size = self.prefill_chunk_size
        c.compute_dtype = capi.COMPUTE_FP32 if self.compute_dtype == "float32" else capi.COMPUTE_BF16
        c.enable_cuda_graphs = int(self.enable_cuda_graphs)
        c.gpu_memory_fraction = self.gpu_memory_fraction
        c.state_slots = self.state_slots
        c.lookahead = int(self.lookahead)
        return c
