"""The Python entry point: load or make a model, then generate.

In the reference's manner (include/imp/imp.h:34-143): a model handle, a
context with engine settings, `generate` for whole requests, and the token
level pair prefill / decode-step, here as `submit` + `step`.  Requests are
lists of token ids (this engine has no tokenizer).

    from imp_b200 import Engine, EngineConfig, GenerateParams
    eng = Engine.from_folder("model_dir", EngineConfig(compute_dtype="bfloat16"))
    outs = eng.generate([[1, 2, 3]], GenerateParams(max_tokens=16, temperature=0.0))
"""
from __future__ import annotations

import itertools
from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence, Tuple

import torch

from ..cache.manager import CacheManager
from ..config.engine_config import EngineConfig
from ..config.model_config import ModelConfig
from ..sampling.sampler import Sampler, SamplingParams
from .loading import load_model, make_cache, random_model
from .model import DecoderModel
from .scheduler import Request, RequestStatus, ScheduledEntry, Scheduler, StepPlan
from .step import StepEntry, Stepper


@dataclass
class GenerateParams:
    """Per-request generation settings; fields and defaults of the reference's
    ImpGenerateParams (include/imp/imp.h:61-85, src/api/imp_api.cpp:76-102) that apply here."""

    temperature: float = 0.7
    top_p: float = 0.9
    top_k: int = 40
    max_tokens: int = 256
    seed: int = -1
    min_p: float = 0.0
    repetition_penalty: float = 1.0
    frequency_penalty: float = 0.0
    presence_penalty: float = 0.0
    repeat_last_n: int = 0
    typical_p: float = 1.0
    dry_multiplier: float = 0.0
    dry_base: float = 1.75
    dry_allowed_length: int = 2
    dry_penalty_last_n: int = 0
    mirostat: int = 0
    mirostat_tau: float = 5.0
    mirostat_eta: float = 0.1
    ignore_eos: bool = False

    def sampling(self) -> SamplingParams:
        return SamplingParams(temperature=self.temperature, top_p=self.top_p, top_k=self.top_k, min_p=self.min_p,
                              repetition_penalty=self.repetition_penalty, frequency_penalty=self.frequency_penalty,
                              presence_penalty=self.presence_penalty, repeat_last_n=self.repeat_last_n,
                              typical_p=self.typical_p, dry_multiplier=self.dry_multiplier, dry_base=self.dry_base,
                              dry_allowed_length=self.dry_allowed_length,
                              dry_penalty_last_n=self.dry_penalty_last_n, mirostat=self.mirostat,
                              mirostat_tau=self.mirostat_tau, mirostat_eta=self.mirostat_eta, seed=self.seed)


@dataclass
class StepOutput:
    rid: Hashable
    token: int
    finished: bool
    status: RequestStatus


@dataclass
class _InFlight:
    """A step that has been queued on the device and whose tokens have not been read yet."""

    plan: StepPlan
    rows: List[Request]              # the requests that get a token, in the order of the sampled tokens
    tokens_dev: Optional[torch.Tensor]   # int32 [len(rows)] on the device
    tokens_host: Optional[torch.Tensor]  # pinned copy of the same, valid once `event` has passed
    status_host: torch.Tensor            # pinned copy of the device status word
    event: torch.cuda.Event
    early: List[StepOutput]          # outputs known at launch (requests the scheduler gave up on)


class Engine:
    """Model + cache + step function + scheduler + sampler on one GPU."""

    def __init__(self, model: DecoderModel, model_config: ModelConfig, config: Optional[EngineConfig] = None):
        self.config = config or EngineConfig()
        self.config.validate()
        self.model = model
        self.model_config = model_config
        cfg = self.config
        rt = model.rt
        if cfg.compute_dtype not in ("bfloat16", "float32") or \
                (cfg.compute_dtype == "float32") != (rt.dtype == torch.float32):
            raise ValueError(f"engine compute_dtype {cfg.compute_dtype} does not match the model's {rt.dtype}")
        self.max_seq_len = min(cfg.max_seq_len, model.plan.max_positions)
        num_pages = self._decide_pages()
        slots = cfg.state_slots or cfg.max_batch_size
        self.cache: CacheManager = make_cache(model, cfg.kv_block_size, num_pages, slots)
        self.stepper = Stepper(model, self.cache, rt, cfg.max_batch_tokens, cfg.max_batch_size, self.max_seq_len,
                               use_cuda_graphs=cfg.enable_cuda_graphs)
        self.scheduler = Scheduler(self.cache, cfg.max_batch_size, cfg.max_batch_tokens, cfg.prefill_chunk_size,
                                   self.max_seq_len)
        self.sampler = Sampler(model.vocab_size, cfg.max_batch_size, rt.device)
        self._inflight: Optional[_InFlight] = None
        # two pinned landing places for (tokens, status): a step in flight and the one launched ahead of it
        self._landing = [(torch.zeros(cfg.max_batch_size, dtype=torch.int32).pin_memory(),
                          torch.zeros(1, dtype=torch.int32).pin_memory()) for _ in range(2)]
        self._landing_turn = 0
        self._ids = itertools.count()
        eos = model_config.eos_token_id
        self.eos_token_ids: Tuple[int, ...] = () if eos is None else (int(eos),)

    # ------------------------------------------------------------ construction
    @classmethod
    def from_folder(cls, model_dir: str, config: Optional[EngineConfig] = None) -> "Engine":
        config = config or EngineConfig()
        mc, model = load_model(model_dir, config.compute_dtype, f"cuda:{config.device_id}")
        return cls(model, mc, config)

    @classmethod
    def from_random(cls, model_config: ModelConfig, config: Optional[EngineConfig] = None, seed: int = 0,
                    std: float = 0.02) -> "Engine":
        config = config or EngineConfig()
        model = random_model(model_config, seed, std, dtype=config.compute_dtype,
                             device=f"cuda:{config.device_id}")
        return cls(model, model_config, config)

    def _decide_pages(self) -> int:
        """Pages per cache group: explicit, or from a token count, or from free memory
        (the reference gives 80% of free memory, clamped to 1-2x the configured worst case:
        src/runtime/engine.cpp:226-243; an explicit block count wins, :531-535)."""
        cfg = self.config
        P = cfg.kv_block_size
        if cfg.kv_cache_max_blocks > 0:
            return cfg.kv_cache_max_blocks
        if cfg.kv_cache_tokens > 0:
            return (cfg.kv_cache_tokens + P - 1) // P
        worst = ((self.max_seq_len + P - 1) // P) * cfg.max_batch_size
        probe = CacheManager(self.model.cache_specs, P, 1, 1)
        per_page = max(1, probe.storage_bytes(torch.empty((), dtype=self.model.rt.dtype).element_size()))
        free, _ = torch.cuda.mem_get_info(self.model.rt.device)
        by_memory = int(free * cfg.gpu_memory_fraction) // per_page
        return max(1, min(worst, by_memory))

    # ---------------------------------------------------------------- requests
    def submit(self, prompt: Sequence[int], params: Optional[GenerateParams] = None,
               rid: Optional[Hashable] = None) -> Request:
        """Queue one request; returns its handle (check `.status` for OUT_OF_MEMORY)."""
        params = params or GenerateParams()
        V = self.model.vocab_size
        for t in prompt:
            if not 0 <= int(t) < V:
                raise ValueError(f"token id {t} outside the vocabulary of {V}")
        req = Request(rid=next(self._ids) if rid is None else rid, prompt=[int(t) for t in prompt],
                      max_tokens=params.max_tokens, params=params.sampling(), eos_token_ids=self.eos_token_ids,
                      ignore_eos=params.ignore_eos)
        return self.scheduler.add(req)

    def has_work(self) -> bool:
        return self.scheduler.has_work() or self._inflight is not None

    # ------------------------------------------------------------------- steps
    def _launch(self, plan: StepPlan, device_tokens: Optional[torch.Tensor] = None,
                early: Optional[List[StepOutput]] = None) -> _InFlight:
        """Queue the plan's batch, its sampling and the copy of the results to pinned memory."""
        entries, rows = [], []
        for e in plan.entries:
            toks = [0] * e.n_tokens if device_tokens is not None else e.request.tokens_slice(e.start, e.n_tokens)
            entries.append(StepEntry(e.request.rid, toks, [e.n_tokens - 1] if e.samples else []))
            if e.samples:
                rows.append(e.request)
        logits = self.stepper.step(entries, device_tokens)
        tokens_dev = tokens_host = None
        land_tokens, land_status = self._landing[self._landing_turn]
        self._landing_turn ^= 1
        if rows:
            # a token launched ahead of the last one's arrival counts as one more output
            ahead = 1 if device_tokens is not None else 0
            tokens_dev = self.sampler.sample_device(
                logits, [r.params for r in rows], [r.seed for r in rows], [len(r.output) + ahead for r in rows],
                [r.all_tokens() for r in rows] if any(r.params.needs_history() for r in rows) else None,
                [r.sampler_state for r in rows])
            tokens_host = land_tokens[:len(rows)]
            tokens_host.copy_(tokens_dev, non_blocking=True)
        land_status.copy_(self.stepper.rt.status, non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        return _InFlight(plan, rows, tokens_dev, tokens_host, land_status, ev, early or [])

    def _finish(self, fl: _InFlight) -> List[StepOutput]:
        """Wait for a queued step, hand its tokens to the scheduler, and report them."""
        fl.event.synchronize()
        code = int(fl.status_host[0])
        if code != 0:
            self.stepper.check_device_status()      # raises with the device's message and clears the word
        outs = list(fl.early)
        live = [r for r in fl.rows if not r.done]   # a request may have finished while this step was under way
        toks = fl.tokens_host.tolist() if fl.rows else []
        sampled = {r.rid: t for r, t in zip(fl.rows, toks)}
        finished = set(id(r) for r in self.scheduler.complete_step(fl.plan, sampled))
        for r in live:
            outs.append(StepOutput(r.rid, sampled[r.rid], id(r) in finished, r.status))
        return outs

    def _plan_ahead(self, fl: _InFlight) -> Optional[StepPlan]:
        """The step after `fl` if it can be decided before `fl`'s tokens are known: every running request
        gets a token from `fl`, none of them ends with it for a reason known in advance (length, context),
        none needs its token on the host to sample the next one, nothing waits for admission, and the pages
        are there.  A request that ends on its end-of-sequence token takes part in one step too many; its
        result is dropped."""
        sch = self.scheduler
        if not self.config.lookahead or not fl.rows or sch.waiting or len(fl.rows) != len(sch.running):
            return None
        if len(fl.plan.entries) != len(fl.rows) or fl.plan.preempted or fl.plan.failed:
            return None
        entries = []
        for e in fl.plan.entries:
            r = e.request
            if r.done or r.params.needs_history() or r.params.mirostat:
                return None
            start = e.start + e.n_tokens
            if len(r.output) + 1 >= r.max_tokens or start + 1 >= self.max_seq_len:
                return None
            entries.append(ScheduledEntry(r, start, 1, True))
        probe = [StepEntry(e.request.rid, [0], [0]) for e in entries]
        if self.stepper.pages_short(probe) > 0:
            return None
        return StepPlan(entries=entries)

    def step(self) -> List[StepOutput]:
        """One engine step: schedule, run the batch, sample, finish.  Returns the new tokens.

        With `lookahead` the step after this one is queued on the device before this one's tokens are
        read (its token ids stay on the device), when `_plan_ahead` allows it; the host's work then
        overlaps the device's.  Every call still returns the tokens of exactly one step."""
        fl = self._inflight
        self._inflight = None
        if fl is None:
            plan = self.scheduler.schedule()
            early = [StepOutput(r.rid, -1, True, r.status) for r in plan.failed]
            if not plan.entries:
                return early
            fl = self._launch(plan, early=early)
        ahead = self._plan_ahead(fl)
        if ahead is not None:
            self._inflight = self._launch(ahead, device_tokens=fl.tokens_dev)
        return self._finish(fl)

    def drain(self) -> List[StepOutput]:
        """Finish a step that was launched ahead, if any (its requests may all have ended already)."""
        fl, self._inflight = self._inflight, None
        return self._finish(fl) if fl is not None else []

    def generate(self, prompts: Sequence[Sequence[int]], params=None) -> List[List[int]]:
        """Generate for every prompt (continuous batching inside); returns the new tokens per prompt.

        `params` is one GenerateParams for all prompts or a list with one per prompt.
        """
        if prompts and isinstance(prompts[0], int):
            raise TypeError("generate takes a list of prompts (each a list of token ids)")
        plist = params if isinstance(params, (list, tuple)) else [params] * len(prompts)
        reqs = [self.submit(p, q) for p, q in zip(prompts, plist)]
        for r in reqs:
            if r.status == RequestStatus.OUT_OF_MEMORY:
                raise MemoryError(f"request {r.rid!r}: prompt plus max_tokens needs more cache pages than the "
                                  f"pool of {self.cache.num_pages} holds")
        while any(not r.done for r in reqs):
            self.step()
        if not self.scheduler.has_work():
            self.drain()
        failed = [r for r in reqs if r.status != RequestStatus.FINISHED]
        if failed:
            raise MemoryError(f"{len(failed)} request(s) ran out of cache pages: "
                              f"{[r.rid for r in failed]}")
        return [list(r.output) for r in reqs]

    # ------------------------------------------------------------- token level
    def step_tokens(self, entries: Sequence[StepEntry]) -> torch.Tensor:
        """Run given tokens as one batch (no scheduling, no sampling); logits of the wanted rows on the host."""
        logits = self.stepper.step(entries)
        out = logits.cpu()
        self.stepper.check_device_status()
        return out

    def end(self, rid: Hashable) -> None:
        """Give back what a `step_tokens` request holds."""
        self.stepper.finish(rid)
