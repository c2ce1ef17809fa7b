"""The scheduler's decisions, driven without a GPU: a stand-in for the step function reserves and
commits pages exactly as the real one does and 'samples' a fixed token."""
import random

import pytest

from imp_b200.cache.manager import CacheManager, PagedKVSpec, StateSpec
from imp_b200.engine.scheduler import FinishReason, Request, RequestStatus, Scheduler
from imp_b200.sampling.sampler import SamplingParams


def make(num_pages=16, page=4, max_batch=4, budget=32, chunk=0, max_seq=256, specs=None, slots=None):
    cache = CacheManager(specs or [PagedKVSpec(2, 16, 0)], page, num_pages, slots or max_batch)
    return cache, Scheduler(cache, max_batch, budget, chunk, max_seq)


def run_step(cache, sched, token=7, log=None):
    """What Engine.step does, minus the GPU: reserve, 'run', commit, sample."""
    plan = sched.schedule()
    sampled = {}
    for e in plan.entries:
        rid = e.request.rid
        if not cache.has(rid):
            cache.add_request(rid)
        assert cache.length(rid) == e.start, "a portion must start where the cache ends"
        cache.reserve(rid, e.start + e.n_tokens)
        cache.commit(rid, e.start + e.n_tokens)
        if e.samples:
            sampled[rid] = token
    cache.check_invariants()
    if log is not None:
        log.append([(e.request.rid, e.start, e.n_tokens, e.samples) for e in plan.entries])
    fin = sched.complete_step(plan, sampled)
    cache.check_invariants()
    return plan, fin


def req(rid, n_prompt, max_tokens=4, **kw):
    return Request(rid, list(range(1, n_prompt + 1)), max_tokens, SamplingParams.greedy(), **kw)


def test_fifo_admission_and_lifecycle():
    cache, s = make()
    for rid, n in (("a", 5), ("b", 9), ("c", 1)):
        s.add(req(rid, n, 3))
    log = []
    plan, fin = run_step(cache, s, log=log)
    # first come first served: a, b, c in arrival order (the reference would sort by length)
    assert log[0] == [("a", 0, 5, True), ("b", 0, 9, True), ("c", 0, 1, True)]
    assert all(len(s.by_id[r].output) == 1 for r in "abc")
    run_step(cache, s, log=log)
    assert log[1] == [("a", 5, 1, True), ("b", 9, 1, True), ("c", 1, 1, True)]
    plan, fin = run_step(cache, s, log=log)
    assert sorted(r.rid for r in fin) == ["a", "b", "c"]
    assert all(r.finish_reason == FinishReason.LENGTH and r.status == RequestStatus.FINISHED for r in fin)
    assert not s.has_work() and cache.free_pages() == 16 and cache.slots.n_free == 4


def test_token_budget_cuts_prompts_into_portions_and_decodes_come_first():
    cache, s = make(num_pages=64, budget=8, chunk=6)
    s.add(req("a", 3, 10))
    log = []
    run_step(cache, s, log=log)
    s.add(req("b", 20, 2))
    for _ in range(5):
        run_step(cache, s, log=log)
    assert log[1] == [("a", 3, 1, True), ("b", 0, 6, False)]     # chunk limit 6
    assert log[2] == [("a", 4, 1, True), ("b", 6, 6, False)]
    assert log[3] == [("a", 5, 1, True), ("b", 12, 6, False)]
    assert log[4] == [("a", 6, 1, True), ("b", 18, 2, True)]     # the rest of the prompt; now it samples
    assert log[5] == [("a", 7, 1, True), ("b", 20, 1, True)]
    cache2, s2 = make(num_pages=64, budget=8, chunk=0)
    s2.add(req("x", 20, 1))
    log2 = []
    for _ in range(3):
        run_step(cache2, s2, log=log2)
    assert log2 == [[("x", 0, 8, False)], [("x", 8, 8, False)], [("x", 16, 4, True)]]   # budget is the limit


def test_batch_size_limit():
    cache, s = make(max_batch=2, num_pages=64)
    for i in range(4):
        s.add(req(i, 3, 2))
    plan, _ = run_step(cache, s)
    assert [e.request.rid for e in plan.entries] == [0, 1]
    plan, fin = run_step(cache, s)
    assert [r.rid for r in fin] == [0, 1]
    plan, _ = run_step(cache, s)
    assert [e.request.rid for e in plan.entries] == [2, 3]


def test_eos_and_ignore_eos_and_context_limit():
    cache, s = make(max_seq=8)
    s.add(req("a", 3, 50, eos_token_ids=(7,)))
    s.add(req("b", 3, 50, eos_token_ids=(7,), ignore_eos=True))
    _, fin = run_step(cache, s, token=7)
    assert [r.rid for r in fin] == ["a"] and fin[0].finish_reason == FinishReason.EOS
    for _ in range(10):
        _, fin = run_step(cache, s, token=7)
        if fin:
            break
    assert fin[0].rid == "b" and fin[0].finish_reason == FinishReason.CONTEXT and fin[0].n_total == 8


def test_any_of_several_end_tokens_finishes_a_request():
    cache, s = make(max_seq=64)
    s.add(req("first", 3, 50, eos_token_ids=(7, 11)))
    s.add(req("second", 3, 50, eos_token_ids=(7, 11)))
    s.add(req("other", 3, 50, eos_token_ids=(5,)))
    _, fin = run_step(cache, s, token=11)               # the second id of the list ends both; 11 is no end token of "other"
    assert sorted(r.rid for r in fin) == ["first", "second"]
    assert all(r.finish_reason == FinishReason.EOS for r in fin)
    _, fin = run_step(cache, s, token=7)
    assert fin == []
    _, fin = run_step(cache, s, token=5)
    assert [r.rid for r in fin] == ["other"] and fin[0].finish_reason == FinishReason.EOS


def test_request_that_can_never_fit_is_refused_when_added():
    cache, s = make(num_pages=4, page=4)          # 16 tokens in all
    r = s.add(req("big", 10, 10))
    assert r.status == RequestStatus.OUT_OF_MEMORY and not s.has_work()
    ok = s.add(req("ok", 10, 6))
    assert ok.status == RequestStatus.WAITING
    with pytest.raises(ValueError):
        s.add(req("ok", 2, 2))
    with pytest.raises(ValueError):
        s.add(Request("e", [], 3))
    with pytest.raises(ValueError):
        s.add(req("long", 300, 2))


def test_preemption_when_pages_run_out_recomputes_later():
    # 6 pages of 4 tokens.  a and b each hold 2 pages after their prompts (7 tokens -> 8 with one output).
    cache, s = make(num_pages=6, page=4, budget=64)
    s.add(req("a", 7, 12))
    s.add(req("b", 7, 12))
    log = []
    plans = []
    for _ in range(40):
        plan, fin = run_step(cache, s, log=log)
        plans.append(plan)
        if not s.has_work():
            break
    a, b = s.by_id["a"], s.by_id["b"]
    assert a.status == RequestStatus.FINISHED and b.status == RequestStatus.FINISHED
    assert len(a.output) == 12 and len(b.output) == 12
    # b (admitted last) was preempted at least once, a never; b restarted from position 0 with its
    # prompt and the tokens it had generated
    assert b.n_preempted >= 1 and a.n_preempted == 0
    pre = next(i for i, p in enumerate(plans) if p.preempted)
    assert plans[pre].preempted[0] is b and all(e.request is not b for e in plans[pre].entries)
    restart = next(step for step in log[pre + 1:] if any(x[0] == "b" for x in step))
    entry = next(x for x in restart if x[0] == "b")
    assert entry[1] == 0                           # recomputed from its start ...
    again = next(x for step in log[pre + 1:] for x in step if x[0] == "b" and x[3])
    assert again[1] + again[2] > 8                 # ... through the tokens it had generated, before it samples again
    assert cache.free_pages() == 6


def test_lone_request_short_of_pages_fails_instead_of_hanging():
    cache, s = make(num_pages=2, page=4, max_seq=64)
    r = s.add(req("a", 6, 2))           # fits: 8 tokens
    assert r.status == RequestStatus.WAITING
    # steal a page so that the pool is smaller than promised
    thief = cache.add_request("thief")
    cache.reserve("thief", 1)
    plans = [run_step(cache, s)[0] for _ in range(3)]
    assert r.status == RequestStatus.OUT_OF_MEMORY and any(p.failed for p in plans) and not s.has_work()


def test_cancel():
    cache, s = make()
    s.add(req("a", 5, 5))
    s.add(req("b", 5, 5))
    run_step(cache, s)
    s.cancel("a")
    assert s.by_id["a"].status == RequestStatus.CANCELLED and not cache.has("a")
    plan, _ = run_step(cache, s)
    assert [e.request.rid for e in plan.entries] == ["b"]


def test_state_slots_limit_admission():
    cache, s = make(specs=[PagedKVSpec(2, 16, 0), StateSpec((4,))], max_batch=4, slots=2, num_pages=64)
    for i in range(3):
        s.add(req(i, 3, 3))
    plan, _ = run_step(cache, s)
    assert [e.request.rid for e in plan.entries] == [0, 1]


def test_random_workloads_finish_and_leave_the_pool_whole():
    rng = random.Random(3)
    for trial in range(30):
        page = rng.choice([1, 4, 16])
        num_pages = rng.randint(8, 40)
        specs = [PagedKVSpec(2, 16, 0)] + ([PagedKVSpec(2, 16, rng.randint(2, 20))] if rng.random() < 0.5 else [])
        chunk = rng.choice([0, 2, 5])
        cache, s = make(num_pages=num_pages, page=page, max_batch=rng.randint(1, 4),
                        budget=rng.randint(4, 24), chunk=chunk, specs=specs, max_seq=num_pages * page)
        reqs = []
        for i in range(rng.randint(1, 8)):
            n = rng.randint(1, max(1, num_pages * page // 3))
            r = s.add(req(i, n, rng.randint(1, 10)))
            if r.status != RequestStatus.OUT_OF_MEMORY:
                reqs.append(r)
        steps = 0
        while s.has_work():
            plan, _ = run_step(cache, s, token=rng.randint(0, 5))
            assert plan.n_tokens <= s.max_batch_tokens and len(plan.entries) <= s.max_batch_size
            if chunk:
                assert all(e.n_tokens <= chunk for e in plan.entries)
            steps += 1
            assert steps < 5000, "scheduler does not make progress"
        assert all(r.status == RequestStatus.FINISHED for r in reqs)
        assert cache.free_pages() == num_pages and cache.slots.n_free == cache.slots.num_pages


def test_long_portions_end_a_step_on_a_multiple_of_256_rows():
    """The products of many rows work in tiles of 256 rows: a portion that does not end its prompt is shortened so that
    the decoding sequences before it and the portion fill whole tiles (64 + 512 rows would be three tiles, 64 + 448 two)."""
    cache, s = make(num_pages=4096, page=16, max_batch=80, budget=576, chunk=512, max_seq=8192)
    for i in range(64):
        s.add(req(f"d{i}", 3, 40))
    log = []
    run_step(cache, s, log=log)                         # the 64 short prompts, whole
    assert len(log[0]) == 64
    s.add(req("long", 3000, 2))
    run_step(cache, s, log=log)
    rows = log[1]
    assert [e[2] for e in rows[:64]] == [1] * 64 and rows[64][0] == "long"
    assert rows[64][2] == 448 and sum(e[2] for e in rows) == 512
    run_step(cache, s, log=log)
    assert log[2][64][1:3] == (448, 448)                # goes on where it stopped, again to a whole tile
    # a portion that ends its prompt is never shortened, and short portions are left alone
    cache2, s2 = make(num_pages=4096, page=16, max_batch=8, budget=600, chunk=512, max_seq=8192)
    s2.add(req("a", 3, 40))
    log2 = []
    run_step(cache2, s2, log=log2)
    s2.add(req("b", 500, 2))
    run_step(cache2, s2, log=log2)
    assert log2[1][1][2] == 500
    cache3, s3 = make(num_pages=64, budget=8, chunk=6)
    s3.add(req("c", 20, 2))
    log3 = []
    run_step(cache3, s3, log=log3)
    assert log3[0][0][2] == 6
