"""The scheduler's decisions, on the host with a fake step function: admission, token budget,
portions, finishing, and what happens when pages run out."""
import random

import pytest

from transformers_neuronx_b200.cache import CacheManager, PagedKVNeed, group_needs
from transformers_neuronx_b200.engine.scheduler import Request, Scheduler


def make(num_pages=8, slots=4, budget=32, max_len=128, portion=None):
    cache = CacheManager(group_needs({0: PagedKVNeed(2, 16)}), 16, num_pages, slots)
    return cache, Scheduler(cache, budget, slots, max_len, max_portion=portion)


def run_step(cache, sched, next_token=lambda req: 7):
    """What the engine does around a plan: take the pages, 'run', sample, commit."""
    plan = sched.schedule()
    for it in plan.items:
        start = cache.append(it.request.rid, it.count)
        assert start == it.start == it.request.computed, "a portion must continue where the cache ends"
    sampled = {it.request.rid: next_token(it.request) for it in plan.items if it.sample}
    done = sched.commit(plan, sampled)
    cache.check()
    return plan, done


def test_refused_at_submit():
    cache, s = make(num_pages=4, max_len=100)
    with pytest.raises(ValueError, match="positions"):
        s.add(Request("a", list(range(90)), 20))
    with pytest.raises(ValueError, match="pages"):
        s.add(Request("b", list(range(60)), 30))      # 89 cached tokens = 6 pages > 4
    with pytest.raises(ValueError, match="empty"):
        s.add(Request("c", [], 3))
    s.add(Request("d", list(range(60)), 5))           # 64 cached tokens = 4 pages: fits exactly


def test_budget_and_portions():
    cache, s = make(num_pages=32, budget=20)
    s.add(Request("a", list(range(50)), 3))
    s.add(Request("b", list(range(9)), 3))
    p, _ = run_step(cache, s)
    assert [(i.request.rid, i.start, i.count, i.sample) for i in p.items] == [("a", 0, 20, False)]
    p, _ = run_step(cache, s)
    assert [(i.request.rid, i.start, i.count) for i in p.items] == [("a", 20, 20)]
    p, _ = run_step(cache, s)      # a's last 10 prompt tokens are sampled after; b gets what is left of the budget
    assert [(i.request.rid, i.start, i.count, i.sample) for i in p.items] == [("a", 40, 10, True), ("b", 0, 9, True)]
    p, _ = run_step(cache, s)      # both decode
    assert [(i.request.rid, i.count, i.sample) for i in p.items] == [("a", 1, True), ("b", 1, True)]
    assert p.n_tokens == 2


def test_decode_goes_before_prompts_and_budget_holds():
    cache, s = make(num_pages=64, slots=4, budget=16, max_len=512)
    s.add(Request("a", list(range(5)), 30))
    run_step(cache, s)
    s.add(Request("b", list(range(100)), 2))
    for _ in range(5):
        p, _ = run_step(cache, s)
        assert p.items[0].request.rid == "a" and p.items[0].count == 1
        assert p.n_tokens <= 16
        assert p.items[1].request.rid == "b" and p.items[1].count == 15


def test_max_portion_and_down_to_one_token():
    cache, s = make(num_pages=64, budget=8, portion=3)
    s.add(Request("a", list(range(7)), 1))
    counts = []
    while s.has_work():
        p, _ = run_step(cache, s)
        counts.append([i.count for i in p.items])
    assert counts == [[3], [3], [1]]


def test_finish_frees_everything():
    cache, s = make(num_pages=8)
    s.add(Request("a", list(range(20)), 2, eos_token_id=2))
    s.add(Request("b", list(range(10)), 50, eos_token_id=2))
    run_step(cache, s)
    _, done = run_step(cache, s, next_token=lambda r: 2 if r.rid == "b" else 7)   # b samples EOS, a reaches its count
    assert sorted(r.rid for r in done) == ["a", "b"]
    assert cache.free_pages() == [8] and cache.slots.num_free == 4 and not s.has_work()
    assert s.running == [] and all(r.finished for r in done)


def test_max_time_ends_a_request_after_a_token():
    """The reference's MaxTimeCriteria (stopping_criteria.py:15-33) is asked after every token whether the
    time is up: a request whose time has passed still gets the token of the step that was running."""
    cache, s = make(num_pages=16)
    a = Request("a", [1, 2, 3], 50, max_time=10.0)
    b = Request("b", [1, 2, 3], 50)
    s.add(a); s.add(b)
    t0 = a.started
    plan = s.schedule()
    for it in plan.items:
        cache.append(it.request.rid, it.count)
    assert s.commit(plan, {"a": 7, "b": 7}, now=t0 + 1.0) == []
    plan = s.schedule()
    for it in plan.items:
        cache.append(it.request.rid, it.count)
    done = s.commit(plan, {"a": 7, "b": 7}, now=t0 + 11.0)
    assert [r.rid for r in done] == ["a"] and a.finish_reason == "time" and a.output == [7, 7]
    assert not b.finished and cache.slots.num_free == 3
    cache.check()


def test_finish_reasons():
    cache, s = make(num_pages=16)
    a, b = Request("a", [1, 2, 3], 2, eos_token_id=2), Request("b", [1, 2, 3], 9, eos_token_id=2)
    s.add(a); s.add(b)
    run_step(cache, s)
    run_step(cache, s, next_token=lambda r: 2 if r.rid == "b" else 7)
    assert (a.finish_reason, b.finish_reason) == ("length", "eos")


def test_eos_ignored_when_asked():
    cache, s = make()
    s.add(Request("a", [1, 2, 3], 4, stop_on_eos=False, eos_token_id=2))
    n = 0
    while s.has_work():
        run_step(cache, s, next_token=lambda r: 2); n += 1
    assert n == 4


def test_admission_waits_for_slots_and_pages():
    cache, s = make(num_pages=4, slots=2, budget=64)
    for rid in "abc":
        s.add(Request(rid, list(range(20)), 4))
    p, _ = run_step(cache, s)
    assert [r.rid for r in p.admitted] == ["a", "b"]           # two slots
    assert [r.rid for r in s.waiting] == ["c"]
    while "c" in [r.rid for r in s.waiting]:
        p, done = run_step(cache, s)
    assert [r.rid for r in p.admitted] == ["c"]                # taken in as soon as one ended


def test_preemption_when_pages_run_out():
    """Two requests decode; the pool cannot hold both to the end.  The one admitted last gives
    everything back, waits, and is computed again from its tokens; all tokens come out."""
    cache, s = make(num_pages=4, slots=4, budget=64, max_len=64)
    s.add(Request("old", list(range(15)), 40))
    s.add(Request("new", list(range(15)), 40))
    seen_preempt = False
    steps = 0
    while s.has_work():
        p, _ = run_step(cache, s, next_token=lambda r: 100 + len(r.output))
        if p.preempted:
            seen_preempt = True
            assert [r.rid for r in p.preempted] == ["new"]     # most recently admitted
            assert s.waiting[0].rid == "new" and s.waiting[0].computed == 0
            assert "new" not in cache
            assert not p.admitted                              # nothing is admitted in the step that preempts
        steps += 1
        assert steps < 500
    assert seen_preempt and s.num_preemptions >= 1
    assert cache.free_pages() == [4]


def test_preempted_request_continues_its_output():
    cache, s = make(num_pages=4, slots=4, budget=64, max_len=64)
    reqs = [Request("old", list(range(15)), 40), Request("new", list(range(15)), 40)]
    for r in reqs:
        s.add(r)
    while s.has_work():
        run_step(cache, s, next_token=lambda r: 100 + len(r.output))
    for r in reqs:
        assert r.output == [100 + i for i in range(40)]       # no token lost or doubled
    assert reqs[1].preemptions >= 1


@pytest.mark.parametrize("seed", range(5))
def test_random_workloads_end(seed):
    rng = random.Random(seed)
    cache, s = make(num_pages=10, slots=3, budget=24, max_len=96)
    reqs = []
    for i in range(12):
        r = Request(i, [rng.randrange(3, 99) for _ in range(rng.randrange(1, 60))], rng.randrange(1, 30), eos_token_id=2)
        s.add(r); reqs.append(r)
    steps = 0
    while s.has_work():
        p, _ = run_step(cache, s, next_token=lambda r: rng.choice([2, 5, 6, 7, 8, 9, 10, 11]))
        assert 0 < p.n_tokens <= 24 and len(s.running) <= 3
        assert len({i.request.rid for i in p.items}) == len(p.items)   # at most one portion per request
        steps += 1
        assert steps < 3000
    assert all(r.finished and 1 <= len(r.output) <= r.max_new_tokens for r in reqs)
    assert cache.free_pages() == [10] and cache.slots.num_free == 3
