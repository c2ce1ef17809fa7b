"""Per-request sampling parameters and the batched sampler over 32-bit logits.

Parameter names and defaults follow the reference's ImpGenerateParams
(include/imp/imp.h:61-85; defaults src/api/imp_api.cpp:76-102, src/runtime/
request.h:40-57): temperature, top_k, top_p, min_p, typical_p, repetition /
frequency / presence penalties with their window `repeat_last_n`, the DRY
penalty, Mirostat v2, seed.  Order of application as in the reference
(src/graph/executor.cu:43-115): penalties, DRY, then either Mirostat v2 (which
takes the temperature and ignores the other filters) or min-p, typical-p and
greedy if temperature <= 0 or top_k == 1, else top-k/top-p at the given
temperature.  The uniform number of a draw is a function of (seed,
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
    typical_p: float = 1.0          # locally typical mass; outside (0, 1) disables
    dry_multiplier: float = 0.0     # DRY penalty scale, 0 disables
    dry_base: float = 1.75
    dry_allowed_length: int = 2     # repeats up to this length cost nothing
    dry_penalty_last_n: int = 0     # how far back DRY looks, 0 = all tokens
    mirostat: int = 0               # 0 off, 2 = Mirostat v2
    mirostat_tau: float = 5.0       # target surprise (bits)
    mirostat_eta: float = 0.1       # learning rate of mu
    seed: int = -1                  # -1 = a fresh random seed per request

    @classmethod
    def greedy(cls) -> "SamplingParams":
        return cls(temperature=0.0, top_p=1.0, top_k=0)

    def is_greedy(self) -> bool:
        return self.mirostat != 2 and (self.temperature <= 0.0 or self.top_k == 1)

    def has_penalties(self) -> bool:
        return self.repetition_penalty != 1.0 or self.frequency_penalty != 0.0 or self.presence_penalty != 0.0

    def has_dry(self) -> bool:
        return self.dry_multiplier > 0.0

    def has_typical(self) -> bool:
        return self.mirostat != 2 and 0.0 < self.typical_p < 1.0

    def needs_history(self) -> bool:
        return self.has_penalties() or self.has_dry()

    def validate(self) -> None:
        if self.top_k < 0:
            raise ValueError("top_k must be >= 0")
        if self.min_p < 0 or self.min_p > 1:
            raise ValueError("min_p must be in [0, 1]")
        if self.repetition_penalty <= 0:
            raise ValueError("repetition_penalty must be positive")
        if self.repeat_last_n < 0:
            raise ValueError("repeat_last_n must be >= 0")
        if self.mirostat not in (0, 2):
            raise ValueError("mirostat must be 0 (off) or 2 (Mirostat v2)")
        if self.dry_multiplier < 0 or self.dry_base <= 0 or self.dry_allowed_length < 0 or self.dry_penalty_last_n < 0:
            raise ValueError("DRY parameters must not be negative (base positive)")


@dataclass
class SamplerState:
    """What a request's sampling carries from token to token: Mirostat's mu (starts at 2 * tau)."""

    mirostat_mu: Optional[float] = None


def dry_penalties(tokens: Sequence[int], multiplier: float, base: float, allowed_length: int,
                  last_n: int = 0) -> dict:
    """The DRY penalty per token id, from the request's tokens so far.

    For every position `pos` in the window, the length of the match between the tokens before
    `pos` and the end of the sequence says how long a repetition would become if `tokens[pos]`
    came next; longer than `allowed_length` costs multiplier * base ** (length - allowed_length),
    the longest match per token counting (src/compute/sampling.cu:826-880).
    """
    n = len(tokens)
    if multiplier <= 0.0 or n < 2:
        return {}
    t = np.asarray(tokens, dtype=np.int64)
    start = max(0, n - last_n) if last_n > 0 else 0
    best: dict = {}
    # only positions preceded by the sequence's last token can match at all
    for pos in (np.flatnonzero(t[start:n - 1] == t[n - 1]) + start + 1).tolist():
        a, b, m = pos - 1, n - 1, 0
        while a >= start and t[a] == t[b]:
            m += 1
            a -= 1
            b -= 1
        if m > allowed_length:
            tok = int(t[pos])
            if m > best.get(tok, 0):
                best[tok] = m
    return {tok: multiplier * float(base) ** (m - allowed_length) for tok, m in best.items()}


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
               steps: Sequence[int], histories: Optional[Sequence[Sequence[int]]] = None,
               states: Optional[Sequence[SamplerState]] = None) -> List[int]:
        """logits [R, V] float32 on the device (modified in place by penalties and filters); returns R token ids.

        `seeds[r]`, `steps[r]` key the uniform number of row r; `histories[r]` are the request's
        tokens so far (prompt and output), used by the penalties and DRY; `states[r]` carries
        Mirostat's mu between calls (needed only for rows that use Mirostat).
        """
        if logits.shape[0] == 0:
            return []
        return self.sample_device(logits, params, seeds, steps, histories, states).tolist()

    def sample_device(self, logits: torch.Tensor, params: Sequence[SamplingParams], seeds: Sequence[int],
                      steps: Sequence[int], histories: Optional[Sequence[Sequence[int]]] = None,
                      states: Optional[Sequence[SamplerState]] = None) -> torch.Tensor:
        """`sample` with the token ids left on the device (int32 [R]).  Without Mirostat rows nothing
        here waits for the device, so the caller can queue more work before it reads the tokens."""
        R = logits.shape[0]
        if R == 0:
            return torch.empty(0, dtype=torch.int32, device=self.device)
        assert len(params) == R and len(seeds) == R and len(steps) == R
        histories = histories or [[] for _ in range(R)]
        if any(p.has_penalties() for p in params):
            self._penalties(logits, params, histories)
        if any(p.has_dry() for p in params):
            self._dry(logits, params, histories)
        if any(p.has_typical() for p in params):
            tp = torch.tensor([[p.typical_p if p.has_typical() else 1.0 for p in params],
                               [p.min_p for p in params]], dtype=torch.float32, device=self.device)
            K.typical_filter(logits, tp[0], tp[1])
        if all(p.is_greedy() for p in params):
            return K.argmax(logits)
        f = np.empty((5, R), dtype=np.float32)
        k = np.empty((2, R), dtype=np.int32)
        miro = [r for r, p in enumerate(params) if p.mirostat == 2]
        if miro and states is None:
            raise ValueError("Mirostat needs the requests' SamplerState objects")
        for r, p in enumerate(params):
            f[0, r] = 0.0 if (p.is_greedy() or p.mirostat == 2) else p.temperature
            f[1, r] = p.top_p if 0.0 < p.top_p < 1.0 else 1.0
            f[2, r] = p.min_p
            f[3, r] = uniform_for(seeds[r], steps[r])
            f[4, r] = 0.0
            k[0, r] = p.top_k
            k[1, r] = 0
        for r in miro:
            st = states[r]
            if st.mirostat_mu is None:
                st.mirostat_mu = 2.0 * params[r].mirostat_tau
            f[4, r] = st.mirostat_mu
            k[1, r] = 1
        fd = torch.from_numpy(f).to(self.device)
        kd = torch.from_numpy(k).to(self.device)
        out = K.sample(logits, fd[0], kd[0], fd[1], fd[2], fd[3])
        if miro:
            temp = torch.tensor([p.temperature for p in params], dtype=torch.float32, device=self.device)
            surprise = torch.zeros(R, dtype=torch.float32, device=self.device)
            K.sample_mirostat(logits, kd[1], temp, fd[4], fd[3], out, surprise)
            sur = surprise.tolist()          # waits for the device: mu is host state
            for r in miro:
                p = params[r]
                states[r].mirostat_mu -= p.mirostat_eta * (sur[r] - p.mirostat_tau)
        return out

    def _dry(self, logits, params, histories) -> None:
        rows: List[int] = []
        toks: List[int] = []
        vals: List[float] = []
        V = logits.shape[1]
        for r, (p, h) in enumerate(zip(params, histories)):
            if not p.has_dry():
                continue
            for tok, v in dry_penalties(h, p.dry_multiplier, p.dry_base, p.dry_allowed_length,
                                        p.dry_penalty_last_n).items():
                if 0 <= tok < V:
                    rows.append(r)
                    toks.append(tok)
                    vals.append(v)
        if not rows:
            return
        it = torch.tensor([rows, toks], dtype=torch.int32, device=self.device)
        K.sparse_subtract(logits, it[0], it[1], torch.tensor(vals, dtype=torch.float32, device=self.device))

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
