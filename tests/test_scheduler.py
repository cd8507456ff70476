"""The scheduler's decisions on the CPU, with the real cache manager and no model: what is
admitted, how prompts are cut under the token budget, that decoding goes first, what
happens when pages run out, and when requests finish."""
import random

import pytest
import torch

from tiny_inference_server_b200.cache import CacheManager
from tiny_inference_server_b200.engine.scheduler import PoolTooSmall, Request, Scheduler
from tiny_inference_server_b200.parts.base import KVSpec
from tiny_inference_server_b200.sampling import SamplingParams


def _sched(num_pages=16, page=4, max_batch=4, budget=16, admission="final", max_context=256, eos=None):
    cache = CacheManager([KVSpec(1, 16), KVSpec(1, 16, lag=1)], {}, page_size=page, num_pages=num_pages,
                         max_slots=max_batch, max_positions=max_context, dtype=torch.float32, device="cpu")
    return Scheduler(cache, max_batch=max_batch, max_tokens_per_step=budget, max_context=max_context,
                     admission=admission, eos_token_id=eos), cache


def _run_step(s, cache, token=1):
    """Plan, 'run' (extend the cache as the step function would), commit."""
    s.admit()
    plan = s.plan_step()
    for e in plan.entries:
        cache.extend(e.request.slot, e.n_tokens)
    s.commit(plan, [token] * sum(1 for e in plan.entries if e.sample))
    cache.check()
    return plan


def _req(n, new=4, **kw):
    return Request(list(range(1, n + 1)), SamplingParams(max_new_tokens=new, **kw))


def test_prompt_is_cut_under_the_token_budget_and_sampled_only_at_its_end():
    s, cache = _sched(budget=5, num_pages=32)
    r = _req(12, new=2)
    s.submit(r)
    sizes = []
    while s.has_work():
        plan = _run_step(s, cache)
        sizes.append([(e.n_tokens, e.sample) for e in plan.entries])
    assert sizes == [[(5, False)], [(5, False)], [(2, True)], [(1, True)]]
    assert r.out_ids() == [1, 1] and r.finish_reason == "length"
    assert cache.drained()


def test_decoding_goes_first_and_prompts_share_what_is_left():
    s, cache = _sched(budget=8, num_pages=64)
    a, b, c = _req(3, new=10), _req(20, new=10), _req(9, new=10)
    s.submit(a)
    _run_step(s, cache)                       # a prefilled, now decoding
    s.submit(b), s.submit(c)
    plan = _run_step(s, cache)
    assert [(e.request, e.n_tokens, e.sample) for e in plan.entries] == [(a, 1, True), (b, 7, False)]
    plan = _run_step(s, cache)
    assert [(e.request, e.n_tokens) for e in plan.entries] == [(a, 1), (b, 7)]
    plan = _run_step(s, cache)
    assert [(e.request, e.n_tokens, e.sample) for e in plan.entries] == [(a, 1, True), (b, 6, True), (c, 1, False)]
    plan = _run_step(s, cache)                # a, b decode; c gets the rest of the budget
    assert [(e.request, e.n_tokens) for e in plan.entries] == [(a, 1), (b, 1), (c, 6)]


def test_final_plan_admits_only_what_fits_at_its_longest():
    # upstream plan="final" (server.py:153-157): never preempts
    s, cache = _sched(num_pages=10, page=4, admission="final", budget=64)
    reqs = [_req(6, new=10) for _ in range(4)]          # each ends at 16 tokens = 4 pages
    for r in reqs:
        s.submit(r)
    s.admit()
    assert len(s.active) == 2 and len(s.queue) == 2
    while s.has_work():
        _run_step(s, cache)
    assert s.preempts == 0 and len(s.finished) == 4 and cache.drained()
    assert s.peak_running == 2


def test_current_plan_admits_more_and_preempts_the_newest():
    # upstream plan="cur" (server.py:158-159) and preempt (server.py:187-193)
    s, cache = _sched(num_pages=5, page=4, admission="cur", budget=64)
    reqs = [_req(3, new=8) for _ in range(4)]           # 1 page each now, 3 pages at the end
    for r in reqs:
        s.submit(r)
    s.admit()
    assert len(s.active) == 4
    order = []
    while s.has_work():
        plan = _run_step(s, cache)
        order += [r.id for r in plan.preempted]
    assert s.preempts > 0 and s.replays > 0
    assert order[0] == reqs[3].id, "the newest request goes first"
    assert all(len(r.out_ids()) == 8 for r in reqs)
    assert cache.drained()
    # a preempted request is fed its prompt and everything it generated, from position 0
    assert max(r.preempted for r in reqs) >= 1


def test_preempted_request_returns_to_the_front_of_the_queue():
    s, cache = _sched(num_pages=2, page=4, admission="cur", budget=64)
    a, b, c = _req(3, new=6), _req(3, new=6), _req(2, new=2)
    s.submit(a), s.submit(b)
    _run_step(s, cache)
    s.submit(c)
    while b.preempted == 0:
        _run_step(s, cache)
    assert s.queue[0] is b and s.queue[1] is c and b.fed == 0 and b.slot is None


def test_a_prompt_that_can_never_fit_is_refused_at_submit():
    s, cache = _sched(num_pages=4, page=4)
    with pytest.raises(PoolTooSmall, match="pages"):
        s.submit(_req(16))
    with pytest.raises(ValueError, match="context"):
        _sched(max_context=8)[0].submit(_req(8))
    s.submit(_req(15))


def test_elastic_portion_when_pages_are_short():
    """A prompt that is fed over several steps finds fewer pages than it wants because the
    decoding requests grew meanwhile: its portion is cut to what fits, it is not sampled
    early, it waits while nothing fits, and when the decoding requests need pages that are
    not there it (the newest) is preempted."""
    s, cache = _sched(num_pages=8, page=4, admission="cur", budget=9)
    a, c = _req(3, new=40), _req(3, new=40)
    s.submit(a), s.submit(c)
    _run_step(s, cache)                        # a, c prefilled: one page each
    b = _req(20, new=1)                        # 5 pages; 6 are free: admitted
    s.submit(b)
    plan = _run_step(s, cache)
    assert [(e.request, e.n_tokens) for e in plan.entries] == [(a, 1), (c, 1), (b, 7)]
    plan = _run_step(s, cache)                 # a and c open their second page
    assert [(e.request, e.n_tokens) for e in plan.entries] == [(a, 1), (c, 1), (b, 7)]
    assert cache.free_pages() == 0
    plan = _run_step(s, cache)                 # b wants 6 tokens, 2 fit the pages it holds
    assert [(e.request, e.n_tokens, e.sample) for e in plan.entries] == [(a, 1, True), (c, 1, True), (b, 2, False)]
    plan = _run_step(s, cache)                 # nothing fits for b: it waits
    assert [(e.request, e.n_tokens) for e in plan.entries] == [(a, 1), (c, 1)] and not plan.preempted
    while not plan.preempted:
        plan = _run_step(s, cache)
    assert plan.preempted == [b] and s.queue[0] is b and b.fed == 0
    assert s.preempts == 1 and s.replays == 1


def test_single_request_too_large_for_the_pool():
    s, cache = _sched(num_pages=2, page=4, admission="cur", budget=64)
    r = _req(5, new=20)
    s.submit(r)
    with pytest.raises(PoolTooSmall, match="single request"):
        for _ in range(30):
            _run_step(s, cache)


def test_finishing_eos_length_context():
    s, cache = _sched(eos=9, num_pages=64, max_context=12, budget=64)
    a, b, c = _req(3, new=5), _req(3, new=50, ignore_eos=True), _req(3, new=50)
    for r in (a, b, c):
        s.submit(r)
    _run_step(s, cache, token=4)
    _run_step(s, cache, token=9)               # end-of-sequence for a and c, b ignores it
    assert a.done and a.finish_reason == "eos" and a.out_ids() == [4, 9]
    assert c.done and not b.done
    while s.has_work():
        _run_step(s, cache, token=9)
    assert b.finish_reason == "context" and len(b.ids) == 12
    assert cache.drained()


def test_random_workloads_drain(seed=0):
    rng = random.Random(seed)
    for trial in range(20):
        s, cache = _sched(num_pages=rng.randint(6, 20), page=rng.choice([2, 4, 8]), max_batch=rng.randint(1, 5),
                          budget=rng.randint(3, 40), admission=rng.choice(["final", "cur"]), max_context=64)
        reqs = []
        for _ in range(rng.randint(1, 12)):
            n = rng.randint(1, 10)
            r = _req(n, new=rng.randint(1, 12))
            try:
                s.submit(r)
                reqs.append(r)
            except PoolTooSmall:
                pass
        steps = 0
        try:
            while s.has_work():
                plan = _run_step(s, cache, token=rng.randint(0, 5))
                assert plan.tokens <= s.max_tokens_per_step
                steps += 1
                assert steps < 5000
        except PoolTooSmall:
            continue
        assert all(r.done for r in reqs) and cache.drained()
        assert all(len(r.out_ids()) == r.params.max_new_tokens or r.finish_reason == "context" for r in reqs)
