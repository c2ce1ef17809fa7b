"""Sampling parameters and the library's batched sampler, for tools and tests.

Parameter names and defaults follow the reference's ImpGenerateParams
(include/imp/imp.h:61-85; defaults src/api/imp_api.cpp:76-102).  The sampler
itself (order of penalties, DRY, Mirostat v2, typical-p, min-p, top-k/top-p;
counter-based uniform numbers) is csrc/host/sampler.cpp over the kernels of
csrc/sampling.cu; `Sampler` here drives it on logits that already live on the
device.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import List, Optional, Sequence

from .. import capi


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

    def to_c(self, max_tokens: int = 256, ignore_eos: bool = False) -> "capi.ImpGenerateParams":
        p = capi.load().imp_generate_params_default()
        for name, _ in capi.ImpGenerateParams._fields_:
            if hasattr(self, name):
                setattr(p, name, getattr(self, name))
        p.max_tokens = max_tokens
        p.ignore_eos = int(ignore_eos)
        return p


@dataclass
class SamplerState:
    """What a request's sampling carries from token to token: Mirostat's mu (starts at 2 * tau)."""

    mirostat_mu: Optional[float] = None


def uniform_for(seed: int, step: int) -> float:
    """The uniform number in [0, 1) of draw `step` of a request seeded with `seed`."""
    lib = capi.load()
    lib.imp_uniform_for.restype = ctypes.c_float
    lib.imp_uniform_for.argtypes = [ctypes.c_uint64, ctypes.c_int64]
    return float(lib.imp_uniform_for(seed, step))


def dry_penalties(tokens: Sequence[int], multiplier: float, base: float, allowed_length: int, last_n: int = 0) -> dict:
    """The DRY penalty per token id, from the request's tokens so far."""
    lib = capi.load()
    lib.imp_dry_penalties.restype = ctypes.c_int
    lib.imp_dry_penalties.argtypes = [ctypes.POINTER(ctypes.c_int32), ctypes.c_int, ctypes.c_float, ctypes.c_float,
                                      ctypes.c_int, ctypes.c_int, ctypes.POINTER(ctypes.c_int32),
                                      ctypes.POINTER(ctypes.c_float), ctypes.c_int]
    toks, n = capi.int32_array([int(t) for t in tokens])
    cap = max(n, 1)
    out_t, out_v = (ctypes.c_int32 * cap)(), (ctypes.c_float * cap)()
    k = lib.imp_dry_penalties(toks, n, multiplier, base, allowed_length, last_n, out_t, out_v, cap)
    return {int(out_t[i]): float(out_v[i]) for i in range(min(k, cap))}


class Sampler:
    """Turns rows of logits on the device into one token per row, through the library's sampler."""

    def __init__(self, vocab_size: int, max_rows: int, device="cuda:0"):
        from ..parts.bench import PartBench
        index = int(str(device).split(":")[1]) if ":" in str(device) else 0
        self.V = vocab_size
        self._bench = PartBench("float32", [], device_id=index)

    def sample(self, logits, params: Sequence[SamplingParams], seeds: Sequence[int], steps: Sequence[int],
               histories: Optional[Sequence[Sequence[int]]] = None,
               states: Optional[Sequence[SamplerState]] = None) -> List[int]:
        """logits [R, V] float32 on the device (a torch tensor; modified in place by penalties and filters)."""
        import torch
        R = logits.shape[0]
        if R == 0:
            return []
        assert logits.dtype == torch.float32 and logits.stride(1) == 1 and logits.is_cuda
        if any(p.mirostat == 2 for p in params) and states is None:
            raise ValueError("Mirostat needs the requests' SamplerState objects")
        lib = capi.load()
        lib.imp_bench_sample.restype = ctypes.c_int
        lib.imp_bench_sample.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_int,
                                         ctypes.POINTER(capi.ImpGenerateParams), ctypes.POINTER(ctypes.c_int64),
                                         ctypes.POINTER(ctypes.c_int64), ctypes.POINTER(ctypes.c_int32),
                                         ctypes.POINTER(ctypes.c_int32), ctypes.POINTER(ctypes.c_float),
                                         ctypes.POINTER(ctypes.c_int32)]
        cp = (capi.ImpGenerateParams * R)(*[p.to_c() for p in params])
        cs = (ctypes.c_int64 * R)(*[int(s) for s in seeds])
        ct = (ctypes.c_int64 * R)(*[int(s) for s in steps])
        histories = histories or [[] for _ in range(R)]
        flat = [int(t) for h in histories for t in h]
        starts = [0]
        for h in histories:
            starts.append(starts[-1] + len(h))
        ch, _ = capi.int32_array(flat)
        chs, _ = capi.int32_array(starts)
        nan = float("nan")
        mu = (ctypes.c_float * R)(*[nan if states is None or states[r].mirostat_mu is None else states[r].mirostat_mu
                                    for r in range(R)])
        out = (ctypes.c_int32 * R)()
        torch.cuda.current_stream(logits.device).synchronize()
        capi.check(lib.imp_bench_sample(self._bench.handle, logits.data_ptr(), logits.stride(0), R, self.V, cp, cs, ct, ch,
                                        chs, mu, out))
        if states is not None:
            for r in range(R):
                if mu[r] == mu[r]:
                    states[r].mirostat_mu = float(mu[r])
        return list(out)
