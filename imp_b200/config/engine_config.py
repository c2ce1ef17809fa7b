"""Engine settings, with the reference's field names where it has them.

`device_id`, `max_batch_size`, `max_seq_len`, `kv_cache_max_blocks`,
`compute_dtype`, `prefill_chunk_size`, `enable_cuda_graphs` come from
include/imp/config.h:11-81 (defaults: src/api/imp_api.cpp:35-72);
`kv_block_size` from src/runtime/engine.h:59.  `max_batch_tokens` (the token
budget of one step) and `lookahead` are this engine's own.
"""
from __future__ import annotations

from dataclasses import dataclass


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
