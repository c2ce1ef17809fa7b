"""The library's scheduler (csrc/host/scheduler.cpp) as a Python object, without a device.

Continuous batching: admission first come first served, prompt portions under
a token budget beside decode tokens, finishing, and preemption by recompute
when pages run out.  The decisions are the library's; this wrapper exists so
that tools and tests can drive them with a stand-in for the step function.
"""
from __future__ import annotations

import ctypes
import json
from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Sequence

from .. import capi
from ..cache.manager import CacheManager
from ..sampling.sampler import SamplingParams
from .engine import FinishReason, RequestStatus


class Request:
    """One generation request as the scheduler sees it; its state is read back from the library."""

    def __init__(self, rid: Hashable, prompt: Sequence[int], max_tokens: int = 256, params: SamplingParams = None,
                 eos_token_ids: Sequence[int] = (), ignore_eos: bool = False):
        self.rid, self.prompt, self.max_tokens = rid, list(prompt), max_tokens
        self.params = params or SamplingParams()
        self.eos_token_ids, self.ignore_eos = tuple(eos_token_ids), ignore_eos
        self._sched = None

    def _j(self):
        return self._sched._info()["requests"][str(self._sched._ids[self.rid])]

    @property
    def status(self) -> RequestStatus:
        return RequestStatus(self._j()["status"])

    @property
    def finish_reason(self) -> FinishReason:
        return FinishReason(self._j()["finish_reason"])

    @property
    def output(self) -> List[int]:
        return self._j()["output"]

    @property
    def n_computed(self) -> int:
        return self._j()["n_computed"]

    @property
    def n_preempted(self) -> int:
        return self._j()["n_preempted"]

    @property
    def n_total(self) -> int:
        return len(self.prompt) + len(self.output)

    @property
    def done(self) -> bool:
        return self.status in (RequestStatus.FINISHED, RequestStatus.CANCELLED, RequestStatus.OUT_OF_MEMORY)

    def all_tokens(self) -> List[int]:
        return self.prompt + self.output


@dataclass
class ScheduledEntry:
    request: Request
    start: int        # index into prompt + output of the first token of this portion
    n_tokens: int
    samples: bool     # the portion ends at the last known token: its last row is sampled


@dataclass
class StepPlan:
    entries: List[ScheduledEntry]
    preempted: List[Request] = field(default_factory=list)
    failed: List[Request] = field(default_factory=list)
    pages: int = 0

    @property
    def n_tokens(self) -> int:
        return sum(e.n_tokens for e in self.entries)


class Scheduler:
    def __init__(self, cache: CacheManager, max_batch_size: int, max_batch_tokens: int, prefill_chunk_size: int = 0,
                 max_seq_len: int = 4096):
        self.cache = cache
        self.max_batch_size, self.max_batch_tokens = max_batch_size, max_batch_tokens
        self.prefill_chunk_size, self.max_seq_len = prefill_chunk_size, max_seq_len
        h = ctypes.c_void_p()
        capi.check(capi.load().imp_scheduler_create(cache.handle, max_batch_size, max_batch_tokens, prefill_chunk_size,
                                                    max_seq_len, ctypes.byref(h)))
        self.handle = h
        self.by_id: Dict[Hashable, Request] = {}
        self._ids = cache._ids   # the cache wrapper's mapping of request ids to integers

    def __del__(self):
        h, self.handle = getattr(self, "handle", None), None
        if h:
            capi.load().imp_scheduler_free(h)

    def _info(self):
        return json.loads(capi.text(capi.load().imp_scheduler_info_json(self.handle)))

    def _name(self, i: int) -> Hashable:
        return self.cache._names[int(i)]

    def add(self, req: Request) -> Request:
        old = self.by_id.get(req.rid)
        if old is not None and not old.done:
            raise ValueError(f"request id {req.rid!r} is already in use")
        toks, n = capi.int32_array([int(t) for t in req.prompt])
        eos, ne = capi.int32_array([int(t) for t in req.eos_token_ids])
        p = req.params.to_c(req.max_tokens, req.ignore_eos)
        status = ctypes.c_int(0)
        capi.check(capi.load().imp_scheduler_add(self.handle, self.cache._id(req.rid, create=True), toks, n, ctypes.byref(p),
                                                 eos, ne, ctypes.byref(status)))
        req._sched = self
        self.by_id[req.rid] = req
        return req

    def cancel(self, rid: Hashable) -> None:
        capi.check(capi.load().imp_scheduler_cancel(self.handle, self.cache._id(rid)))

    def has_work(self) -> bool:
        j = self._info()
        return bool(j["waiting"] or j["running"])

    @property
    def waiting(self) -> List[Request]:
        return [self.by_id[self._name(i)] for i in self._info()["waiting"]]

    @property
    def running(self) -> List[Request]:
        return [self.by_id[self._name(i)] for i in self._info()["running"]]

    def schedule(self) -> StepPlan:
        j = capi.call_json(capi.load().imp_scheduler_schedule, self.handle, kind=None)
        req = lambda i: self.by_id[self._name(i)]   # noqa: E731
        return StepPlan([ScheduledEntry(req(e["id"]), e["start"], e["n_tokens"], e["samples"]) for e in j["entries"]],
                        [req(i) for i in j["preempted"]], [req(i) for i in j["failed"]], j["pages"])

    def complete_step(self, plan: StepPlan, sampled: Dict[Hashable, int]) -> List[Request]:
        toks, n = capi.int32_array([int(sampled[e.request.rid]) for e in plan.entries if e.samples])
        out = ctypes.c_char_p()
        capi.check(capi.load().imp_scheduler_complete(self.handle, toks, n, ctypes.byref(out)))
        return [self.by_id[self._name(i)] for i in json.loads(out.value.decode())]
