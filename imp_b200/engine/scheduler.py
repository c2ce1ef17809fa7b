"""Continuous batching: admission, prompt portions under a token budget, decode, finish.

Compared with the reference (src/runtime/scheduler.cpp:16-112, src/runtime/
engine.cpp:1074-1515, 1528-2050):

* admission is first come first served (the reference sorts the queue by
  prompt length, scheduler.cpp:32-38), so the same arrivals always give the
  same batches;
* one step holds decode tokens and prompt portions together, under
  `max_batch_tokens` (the reference runs every prefilling request in a forward
  pass of its own and has no per-step token budget, engine.cpp:1101-1120);
* pages are reserved portion by portion, not for the whole prompt up front
  (scheduler.cpp:48-80);
* when pages run out, nothing is evicted silently (the reference frees the
  least recently used sequence's pages without telling its request, which is
  then cancelled at its next step: engine.cpp:1541-1553, kv_cache_manager.cpp:
  158-170).  Instead the scheduler *preempts* the request that was admitted
  last: its pages and slot are returned, and it goes back to the head of the
  waiting queue to be recomputed later from its prompt plus the tokens it has
  generated so far.  A request that could not fit even with the whole pool to
  itself is refused when it is added (status OUT_OF_MEMORY).

The scheduler only decides; it talks to the cache manager for page counts and
to nothing else, so it runs without a GPU.
"""
from __future__ import annotations

import enum
from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, Hashable, List, Optional, Sequence

from ..cache.manager import CacheManager
from ..sampling.sampler import SamplerState, SamplingParams, resolve_seed


class RequestStatus(enum.Enum):
    WAITING = "waiting"
    RUNNING = "running"
    FINISHED = "finished"
    CANCELLED = "cancelled"
    OUT_OF_MEMORY = "out_of_memory"


class FinishReason(enum.Enum):
    EOS = "eos"
    LENGTH = "length"          # max_tokens reached
    CONTEXT = "context"        # the sequence reached max_seq_len
    NONE = "none"


@dataclass
class Request:
    """One generation request (the reference's Request: src/runtime/request.h:32-74)."""

    rid: Hashable
    prompt: List[int]
    max_tokens: int = 256
    params: SamplingParams = field(default_factory=SamplingParams)
    eos_token_ids: Sequence[int] = ()
    ignore_eos: bool = False
    output: List[int] = field(default_factory=list)
    status: RequestStatus = RequestStatus.WAITING
    finish_reason: FinishReason = FinishReason.NONE
    n_computed: int = 0            # tokens of prompt+output whose keys/state are in the cache
    seed: int = 0                  # resolved sampling seed
    n_preempted: int = 0
    sampler_state: SamplerState = field(default_factory=SamplerState)

    def all_tokens(self) -> List[int]:
        return self.prompt + self.output

    def tokens_slice(self, start: int, n: int) -> List[int]:
        """Tokens [start, start+n) of prompt followed by output, without joining the two lists."""
        np_ = len(self.prompt)
        if start >= np_:
            return self.output[start - np_: start - np_ + n]
        if start + n <= np_:
            return self.prompt[start: start + n]
        return self.prompt[start:] + self.output[: start + n - np_]

    @property
    def n_total(self) -> int:
        return len(self.prompt) + len(self.output)

    @property
    def done(self) -> bool:
        return self.status in (RequestStatus.FINISHED, RequestStatus.CANCELLED, RequestStatus.OUT_OF_MEMORY)


@dataclass
class ScheduledEntry:
    request: Request
    start: int        # index into all_tokens() of the first token of this portion
    n_tokens: int
    samples: bool     # the portion ends at the last known token: its last row is sampled


@dataclass
class StepPlan:
    entries: List[ScheduledEntry]
    preempted: List[Request] = field(default_factory=list)
    failed: List[Request] = field(default_factory=list)
    pages: int = 0    # pages the entries so far will take from the pool

    @property
    def n_tokens(self) -> int:
        return sum(e.n_tokens for e in self.entries)


class Scheduler:
    def __init__(self, cache: CacheManager, max_batch_size: int, max_batch_tokens: int,
                 prefill_chunk_size: int = 0, max_seq_len: int = 4096):
        self.cache = cache
        self.max_batch_size = max_batch_size
        self.max_batch_tokens = max_batch_tokens
        self.prefill_chunk_size = prefill_chunk_size
        self.max_seq_len = max_seq_len
        self.waiting: Deque[Request] = deque()
        self.running: List[Request] = []   # in admission order
        self.by_id: Dict[Hashable, Request] = {}

    # ----------------------------------------------------------------- arrivals
    def add(self, req: Request) -> Request:
        if req.rid in self.by_id and not self.by_id[req.rid].done:
            raise ValueError(f"request id {req.rid!r} is already in use")
        if not req.prompt:
            raise ValueError("a request needs at least one prompt token")
        if req.max_tokens <= 0:
            raise ValueError("max_tokens must be positive")
        if len(req.prompt) >= self.max_seq_len:
            raise ValueError(f"prompt of {len(req.prompt)} tokens leaves no room under max_seq_len {self.max_seq_len}")
        req.params.validate()
        req.seed = resolve_seed(req.params.seed)
        self.by_id[req.rid] = req
        most = min(len(req.prompt) + req.max_tokens, self.max_seq_len)
        if self._pages_for_whole(most) > self.cache.num_pages:
            req.status = RequestStatus.OUT_OF_MEMORY
            return req
        req.status = RequestStatus.WAITING
        self.waiting.append(req)
        return req

    def _pages_for_whole(self, n_tokens: int) -> int:
        """Pages of the hungriest group for a request of n_tokens with the pool to itself."""
        P = self.cache.page_size
        need = 0
        for g in self.cache.paged:
            if g.spec.window > 0:
                # live span is at most window + one portion; count the window plus one page of slack
                span = min(n_tokens, g.spec.window + max(self.prefill_chunk_size, 1) + P)
                need = max(need, (span + P - 1) // P)
            else:
                need = max(need, (n_tokens + P - 1) // P)
        return need

    def cancel(self, rid: Hashable) -> None:
        req = self.by_id.get(rid)
        if req is None or req.done:
            return
        if req in self.running:
            self.running.remove(req)
            self._release(req)
        elif req in self.waiting:
            self.waiting.remove(req)
        req.status = RequestStatus.CANCELLED

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    # ----------------------------------------------------------------- planning
    def _release(self, req: Request) -> None:
        if self.cache.has(req.rid):
            self.cache.release(req.rid)
        req.n_computed = 0

    def _preempt(self, victim: Request, plan: StepPlan) -> None:
        """Return `victim`'s pages and slot; it waits at the head of the queue to be recomputed."""
        self.running.remove(victim)
        plan.entries = [e for e in plan.entries if e.request is not victim]
        self._release(victim)
        plan.pages = sum(self._pages_needed(e.request, e.start + e.n_tokens) for e in plan.entries)
        victim.status = RequestStatus.WAITING
        victim.n_preempted += 1
        self.waiting.appendleft(victim)
        plan.preempted.append(victim)

    def _pages_needed(self, req: Request, new_len: int) -> int:
        if self.cache.has(req.rid):
            return self.cache.pages_needed(req.rid, new_len)
        return max((g.pages_needed_n(0, 0, new_len) for g in self.cache.paged), default=0)

    def _free_after(self, plan: StepPlan) -> int:
        """Free pages left once everything already in the plan has been reserved."""
        return self.cache.free_pages() - plan.pages

    def _largest_fit(self, req: Request, n: int, free: int) -> int:
        """The most tokens <= n that `req` can take next with `free` pages."""
        P = self.cache.page_size
        room_in_last_page = (-req.n_computed) % P if self.cache.has(req.rid) else 0
        fit = min(n, max(free, 0) * P + room_in_last_page)
        while fit >= 1 and self._pages_needed(req, req.n_computed + fit) > free:
            fit -= 1  # windowed groups can need a page more than the simple count
        return max(fit, 0)

    def _serve_running(self, req: Request, plan: StepPlan, budget: int, chunk: int) -> int:
        """Plan the next tokens of a running request; returns how many tokens it got."""
        remaining = req.n_total - req.n_computed
        decoding = remaining == 1
        n = 1 if decoding else min(remaining, chunk, budget)
        while True:
            free = self._free_after(plan)
            if self._pages_needed(req, req.n_computed + n) <= free:
                break
            if not decoding:
                fit = self._largest_fit(req, n, free)
                if fit >= 1:
                    n = fit
                    break
                if req is not self.running[0]:
                    return 0  # a younger prompt waits for pages; the oldest request always goes on
            victim = self.running[-1]
            if victim is req:
                if len(self.running) == 1:
                    # alone with the whole pool and still short of pages: it cannot go on
                    self.running.remove(req)
                    self._release(req)
                    req.status = RequestStatus.OUT_OF_MEMORY
                    plan.failed.append(req)
                else:
                    self._preempt(req, plan)
                return 0
            self._preempt(victim, plan)
        plan.pages += self._pages_needed(req, req.n_computed + n)
        plan.entries.append(ScheduledEntry(req, req.n_computed, n, req.n_computed + n == req.n_total))
        return n

    def schedule(self) -> StepPlan:
        """Decide the next step's batch: decode tokens first, then portions of running prompts,
        then new requests.  Touches the cache only to release what it preempts."""
        plan = StepPlan(entries=[])
        budget = self.max_batch_tokens
        chunk = self.prefill_chunk_size if self.prefill_chunk_size > 0 else self.max_batch_tokens

        for decoding in (True, False):
            for req in list(self.running):
                if req not in self.running or budget <= 0:
                    continue
                if ((req.n_total - req.n_computed) == 1) != decoding:
                    continue
                budget -= self._serve_running(req, plan, budget, chunk)

        P = self.cache.page_size
        while self.waiting and budget > 0 and len(self.running) < self.max_batch_size:
            req = self.waiting[0]
            if req in plan.preempted:
                break  # just preempted for lack of pages: not again in the same step
            new_in_plan = sum(1 for e in plan.entries if not self.cache.has(e.request.rid))
            if self.cache.slots.n_free - new_in_plan <= 0:
                break
            n = min(req.n_total, chunk, budget)
            free = self._free_after(plan)
            # Keep one page in hand per running request so that decoding can go on.
            usable = free - len(self.running) if self.running else free
            if self._pages_needed(req, n) > usable:
                n = min(n, max(usable, 0) * P)
                if n < 1:
                    break
            self.waiting.popleft()
            req.status = RequestStatus.RUNNING
            req.n_computed = 0
            self.running.append(req)
            plan.pages += self._pages_needed(req, n)
            plan.entries.append(ScheduledEntry(req, 0, n, n == req.n_total))
            budget -= n
        return plan

    # ------------------------------------------------------------------ results
    def complete_step(self, plan: StepPlan, sampled: Dict[Hashable, int]) -> List[Request]:
        """Record a finished step: advance lengths, append sampled tokens, finish requests.

        `sampled` maps the request id of every entry with `samples` to its new token.
        Returns the requests that finished in this step (their cache has been released).
        """
        finished = []
        for e in plan.entries:
            req = e.request
            if req.done:
                continue    # finished or cancelled while this step was already under way
            req.n_computed = e.start + e.n_tokens
            if not e.samples:
                continue
            tok = int(sampled[req.rid])
            req.output.append(tok)
            reason = FinishReason.NONE
            if not req.ignore_eos and tok in req.eos_token_ids:
                reason = FinishReason.EOS
            elif len(req.output) >= req.max_tokens:
                reason = FinishReason.LENGTH
            elif req.n_total >= self.max_seq_len:
                reason = FinishReason.CONTEXT
            if reason is not FinishReason.NONE:
                req.status = RequestStatus.FINISHED
                req.finish_reason = reason
                self.running.remove(req)
                self._release(req)
                finished.append(req)
        return finished
