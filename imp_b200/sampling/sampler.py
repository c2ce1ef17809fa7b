"""Per-request sampling parameters and the batched sampler over 32-bit logits.

Parameter names and defaults follow the reference's ImpGenerateParams
(include/imp/imp.h:61-85; defaults src/api/imp_api.cpp:76-102) for the filters
this engine implements: temperature, top_k, top_p, min_p, repetition /
frequency / presence penalties with their window `repeat_last_n`, seed.  Order
of application as in the reference (src/graph/executor.cu:43-115): penalties,
then min-p, then greedy if temperature <= 0 or top_k == 1, else top-k/top-p at
the given temperature.  The uniform number of a draw is a function of (seed,
step index of the request) alone, so a request's tokens do not depend on the
batch it was sampled in; the reference re-seeds its generator with the same
seed at every call (src/compute/sampling.cu:541-543) and so repeats one draw.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import List, Optional, Sequence

import numpy as np
import torch

from ..ops import kernels as K


@dataclass
class SamplingParams:
    temperature: float = 0.7        # <= 0 means greedy
    top_p: float = 0.9              # nucleus mass; >= 1 or <= 0 disables
    top_k: int = 40                 # 0 disables; 1 means greedy
    min_p: float = 0.0              # 0 disables
    repetition_penalty: float = 1.0
    frequency_penalty: float = 0.0
    presence_penalty: float = 0.0
    repeat_last_n: int = 0          # penalty window over the request's tokens, 0 = all
    seed: int = -1                  # -1 = a fresh random seed per request

    @classmethod
    def greedy(cls) -> "SamplingParams":
        return cls(temperature=0.0, top_p=1.0, top_k=0)

    def is_greedy(self) -> bool:
        return self.temperature <= 0.0 or self.top_k == 1

    def has_penalties(self) -> bool:
        return self.repetition_penalty != 1.0 or self.frequency_penalty != 0.0 or self.presence_penalty != 0.0

    def validate(self) -> None:
        if self.top_k < 0:
            raise ValueError("top_k must be >= 0")
        if self.min_p < 0 or self.min_p > 1:
            raise ValueError("min_p must be in [0, 1]")
        if self.repetition_penalty <= 0:
            raise ValueError("repetition_penalty must be positive")
        if self.repeat_last_n < 0:
            raise ValueError("repeat_last_n must be >= 0")


_MASK = (1 << 64) - 1


def resolve_seed(seed: int) -> int:
    """A concrete 63-bit seed: `seed` itself, or fresh randomness for -1."""
    if seed is None or seed < 0:
        return int.from_bytes(os.urandom(8), "little") >> 1
    return int(seed)


def uniform_for(seed: int, step: int) -> float:
    """The uniform number in [0, 1) of draw `step` of a request seeded with `seed` (splitmix64)."""
    z = (seed * 0x9E3779B97F4A7C15 + (step + 1) * 0xBF58476D1CE4E5B9) & _MASK
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK
    z ^= z >> 31
    return (z >> 40) / float(1 << 24)


class Sampler:
    """Turns the logits rows of a step into one token per row."""

    def __init__(self, vocab_size: int, max_rows: int, device):
        self.V, self.max_rows, self.device = vocab_size, max_rows, device
        self._counts: Optional[torch.Tensor] = None  # [max_rows, V] int32, made on first use of penalties

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams], seeds: Sequence[int],
               steps: Sequence[int], histories: Optional[Sequence[Sequence[int]]] = None) -> List[int]:
        """logits [R, V] float32 on the device (modified in place by penalties); returns R token ids.

        `seeds[r]`, `steps[r]` key the uniform number of row r; `histories[r]` are the request's
        tokens so far (prompt and output), used by the penalties.
        """
        R = logits.shape[0]
        if R == 0:
            return []
        assert len(params) == R and len(seeds) == R and len(steps) == R
        if any(p.has_penalties() for p in params):
            self._penalties(logits, params, histories or [[] for _ in range(R)])
        if all(p.is_greedy() for p in params):
            return K.argmax(logits).tolist()
        f = np.empty((4, R), dtype=np.float32)
        k = np.empty(R, dtype=np.int32)
        for r, p in enumerate(params):
            f[0, r] = 0.0 if p.is_greedy() else p.temperature
            f[1, r] = p.top_p if 0.0 < p.top_p < 1.0 else 1.0
            f[2, r] = p.min_p
            f[3, r] = uniform_for(seeds[r], steps[r])
            k[r] = p.top_k
        fd = torch.from_numpy(f).to(self.device)
        kd = torch.from_numpy(k).to(self.device)
        return K.sample(logits, fd[0], kd, fd[1], fd[2], fd[3]).tolist()

    def _penalties(self, logits, params, histories) -> None:
        R = logits.shape[0]
        if self._counts is None or self._counts.shape[0] < R:
            self._counts = torch.empty((max(R, self.max_rows), self.V), dtype=torch.int32, device=self.device)
        flat: List[int] = []
        start = [0]
        max_hist = 0
        for p, h in zip(params, histories):
            h = list(h) if p.has_penalties() else []
            if p.repeat_last_n > 0:
                h = h[-p.repeat_last_n:]
            flat.extend(h)
            start.append(len(flat))
            max_hist = max(max_hist, len(h))
        if max_hist == 0:
            return
        hist = torch.tensor(flat, dtype=torch.int32, device=self.device)
        hs = torch.tensor(start, dtype=torch.int32, device=self.device)
        pen = torch.tensor([[p.repetition_penalty for p in params], [p.frequency_penalty for p in params],
                            [p.presence_penalty for p in params]], dtype=torch.float32, device=self.device)
        K.apply_penalties(logits, hist, hs, max_hist, pen[0], pen[1], pen[2], self._counts)
