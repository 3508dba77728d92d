"""The scheduler's decisions with a fake step function (no GPU): admission, token
budget, portions, decode first, finishing, and what happens when pages run out."""
import random

import pytest
import torch

from batchspec_b200.cache import CacheManager
from batchspec_b200.engine.scheduler import Scheduler
from batchspec_b200.engine.sequence import Sequence, Status
from batchspec_b200.models.decoder import CacheNeed
from batchspec_b200.parts import CacheSpec

FULL = CacheSpec("full", (1, 16))


def make(num_pages=64, page_size=4, max_concurrency=4, budget=16, chunk=8, max_len=1000, eos=(), ignore_eos=False):
    cache = CacheManager([CacheNeed(FULL, None, None)], page_size, num_pages, max_concurrency, torch.float32, "cpu",
                         allocate=False)
    return cache, Scheduler(cache, max_concurrency, budget, chunk, max_len, eos, ignore_eos)


def fake_step(cache, work, token_of=lambda s: 1000 + len(s.output_ids)):
    """What the engine does around the model: reserve, commit, hand back a token."""
    assert cache.can_reserve([(cache.length(w.seq.seq_id), w.n_tokens) for w in work])
    out = {}
    for w in work:
        assert cache.length(w.seq.seq_id) == w.start == w.seq.num_computed
        cache.reserve(w.seq.seq_id, w.n_tokens)
        cache.commit(w.seq.seq_id, w.n_tokens)
        if w.wants_token:
            out[w.seq.seq_id] = token_of(w.seq)
    cache.check_invariants()
    return out


def run(cache, sched, max_steps=10000, **kw):
    plans = []
    while not sched.is_done():
        work = sched.plan()
        if not work:
            assert sched.is_done(), "a scheduler with unfinished requests must always find work"
            break
        plans.append([(w.seq.seq_id, w.start, w.n_tokens, w.wants_token) for w in work])
        sched.process_results(work, fake_step(cache, work, **kw))
        assert len(plans) < max_steps
    return plans


def test_budget_portions_and_decode_first():
    cache, sched = make(budget=10, chunk=8)
    sched.add_sequences([Sequence(0, list(range(13)), 3), Sequence(1, list(range(5)), 2)])
    plans = run(cache, sched)
    assert plans[0] == [(0, 0, 8, False), (1, 0, 2, False)]             # budget 10 = 8 + 2
    assert plans[1] == [(0, 8, 5, True), (1, 2, 3, True)]              # both prompts end: tokens wanted
    assert plans[2] == [(0, 13, 1, True), (1, 5, 1, True)]             # decode
    assert all(sum(n for _, _, n, _ in p) <= 10 for p in plans)
    s0, s1 = sorted(sched.completed, key=lambda s: s.seq_id)
    assert s0.output_ids == [1000, 1001, 1002] and s0.finish_reason == "length"
    assert s1.output_ids == [1000, 1001] and cache.groups[0].pool.num_free == 64


def test_decode_entries_come_before_prompt_portions():
    cache, sched = make(budget=6, chunk=8, max_concurrency=3)
    sched.add_sequences([Sequence(0, [1, 2], 5)])
    w = sched.plan()
    sched.process_results(w, fake_step(cache, w))
    sched.add_sequences([Sequence(1, list(range(20)), 2)])
    w = sched.plan()
    assert [(x.seq.seq_id, x.n_tokens) for x in w] == [(0, 1), (1, 5)]   # the decode token first, rest of the budget


def test_fifo_admission_and_concurrency_cap():
    cache, sched = make(max_concurrency=2, budget=100, chunk=100)
    sched.add_sequences([Sequence(i, [1] * 3, 2) for i in range(5)])
    plans = run(cache, sched)
    assert all(len(p) <= 2 for p in plans)
    first_seen = []
    for p in plans:
        for sid, *_ in p:
            if sid not in first_seen:
                first_seen.append(sid)
    assert first_seen == [0, 1, 2, 3, 4]


def test_eos_stops_even_the_first_token_unless_ignored():
    cache, sched = make(eos=(7,))
    sched.add_sequences([Sequence(0, [1, 2, 3], 10)])
    run(cache, sched, token_of=lambda s: 7)
    assert sched.completed[0].output_ids == [7] and sched.completed[0].finish_reason == "eos"
    cache, sched = make(eos=(7,), ignore_eos=True)
    sched.add_sequences([Sequence(0, [1, 2, 3], 4)])
    run(cache, sched, token_of=lambda s: 7)
    assert sched.completed[0].output_ids == [7] * 4 and sched.completed[0].finish_reason == "length"


def test_context_limit_and_requests_that_can_never_run():
    cache, sched = make(max_len=6, num_pages=3, page_size=4)
    sched.add_sequences([Sequence(0, [1] * 4, 50), Sequence(1, [1] * 6, 5), Sequence(2, [], 5), Sequence(3, [1], 0)])
    failed = {s.seq_id: s.finish_reason for s in sched.completed}
    assert set(failed) == {1, 2, 3} and "context" in failed[1]
    run(cache, sched)
    s0 = [s for s in sched.completed if s.seq_id == 0][0]
    assert s0.status is Status.COMPLETE and s0.finish_reason == "context" and s0.total_len == 6
    cache, sched = make(num_pages=2, page_size=4)
    sched.add_sequences([Sequence(0, [1] * 9, 5)])
    assert sched.completed[0].status is Status.FAILED and "pool" in sched.completed[0].finish_reason


def test_a_request_that_outgrows_the_whole_pool_ends_with_what_it_has():
    cache, sched = make(num_pages=3, page_size=4, budget=32, chunk=32)
    sched.add_sequences([Sequence(0, [1] * 10, 50)])
    run(cache, sched)
    s = sched.completed[0]
    assert s.status is Status.COMPLETE and s.finish_reason == "cache" and s.total_len == 13
    assert sched.num_preemptions == 0 and cache.groups[0].pool.num_free == 3


def test_admission_waits_for_pages():
    cache, sched = make(num_pages=4, page_size=4, budget=32, chunk=32)
    sched.add_sequences([Sequence(0, [1] * 12, 2), Sequence(1, [1] * 8, 2)])
    w = sched.plan()
    assert [x.seq.seq_id for x in w] == [0], "the second prompt's portion does not fit beside the first"
    sched.process_results(w, fake_step(cache, w))
    plans = run(cache, sched)
    assert sched.num_preemptions == 0 and {s.seq_id for s in sched.completed} == {0, 1}


def test_running_out_of_pages_preempts_the_latest_and_recomputes():
    # two requests that each grow to 4 pages in a pool of 6: one must give way
    cache, sched = make(num_pages=6, page_size=4, budget=32, chunk=32, max_concurrency=2)
    sched.add_sequences([Sequence(0, [1] * 7, 9), Sequence(1, [2] * 7, 9)])
    plans = run(cache, sched)
    assert sched.num_preemptions >= 1
    a, b = sorted(sched.completed, key=lambda s: s.seq_id)
    assert a.num_preemptions == 0 and b.num_preemptions >= 1, "the most recently admitted request gives way"
    assert a.output_ids == [1000 + i for i in range(9)] and b.output_ids == [1000 + i for i in range(9)]
    # after the preemption request 1 fed prompt + generated tokens again, from position 0
    restarts = [p for p in plans for (sid, start, n, _) in p if sid == 1 and start == 0]
    assert len(restarts) >= 2
    assert cache.groups[0].pool.num_free == 6


@pytest.mark.parametrize("seed", range(5))
def test_random_workloads_finish_with_clean_books(seed):
    rng = random.Random(seed)
    cache, sched = make(num_pages=rng.randrange(8, 24), page_size=rng.choice([2, 4, 8]),
                        max_concurrency=rng.randrange(1, 5), budget=rng.randrange(4, 24), chunk=rng.randrange(2, 12),
                        max_len=64, eos=(3,))
    seqs = [Sequence(i, [rng.randrange(10) for _ in range(rng.randrange(1, 30))], rng.randrange(1, 12)) for i in range(25)]
    sched.add_sequences(seqs)
    run(cache, sched, token_of=lambda s: rng.randrange(10))
    assert len(sched.completed) == 25 and not sched.running and not sched.waiting_queue
    for s in sched.completed:
        if s.status is Status.COMPLETE:
            assert 1 <= len(s.output_ids) <= s.max_new_tokens and s.total_len <= 64
            assert s.finish_reason in ("eos", "length", "context", "cache")
            if s.finish_reason == "cache":
                assert cache.pages_needed(0, s.total_len)[0] > cache.groups[0].pool.num_pages
            if s.finish_reason == "eos":
                assert s.output_ids[-1] == 3 and 3 not in s.output_ids[:-1]
    assert cache.groups[0].pool.num_free == cache.groups[0].pool.num_pages
    cache.check_invariants()


def test_a_windows_small_pool_does_not_refuse_a_long_prompt():
    """A group of layers that reads a window of keys gives pages back as the window passes: its pool need not hold
    a whole request.  A prompt longer than that pool is admitted, fed in portions and decoded to its end; only a
    pool that cannot hold the first portion, or the window plus the token in flight, refuses it."""
    win = CacheSpec("window", (1, 16), window=6)
    def build(win_pages):
        cache = CacheManager([CacheNeed(FULL, None, None), CacheNeed(win, None, None)], 4, [64, win_pages], 2,
                             torch.float32, "cpu", allocate=False)
        return cache, Scheduler(cache, 2, 8, 8, 1000)
    cache, sched = build(5)                      # 20 tokens' worth of pages for the window's group
    sched.add_sequences([Sequence(0, list(range(50)), 9), Sequence(1, list(range(31)), 4)])
    run(cache, sched)
    done = sorted(sched.completed, key=lambda s: s.seq_id)
    assert [s.finish_reason for s in done] == ["length", "length"] and [len(s.output_ids) for s in done] == [9, 4]
    assert all(g.pool.num_held == 0 for g in cache.groups) and cache.groups[1].pool.high_water <= 5
    cache, sched = build(3)                      # later portions shrink to the room there is
    sched.add_sequences([Sequence(0, list(range(50)), 9)])
    run(cache, sched)
    assert sched.completed[0].finish_reason == "length" and cache.groups[1].pool.high_water <= 3
    for pages in (2, 1):                         # window 6 and a token in pages of 4 can take 3; the first portion 2
        cache, sched = build(pages)
        sched.add_sequences([Sequence(0, list(range(50)), 9)])
        assert sched.completed[0].status is Status.FAILED and "more pages" in sched.completed[0].finish_reason


@pytest.mark.parametrize("seed", range(8))
def test_random_workloads_with_a_windows_pool_finish_with_clean_books(seed):
    """Two groups with pools of their own, the window's one tight: every request that is accepted runs to its end
    (none is refused or cut short for the window's pool, which only has to hold the window and a portion), the
    window's pool never holds more than it has, and all pages come back."""
    rng = random.Random(100 + seed)
    page, window = rng.choice([2, 4, 8]), rng.randrange(3, 20)
    chunk, conc = rng.randrange(2, 12), rng.randrange(1, 5)
    budget = rng.randrange(max(4, conc), 24)
    first = min(chunk, budget)
    win_pages = max((window + page - 1) // page + 1, -(-first // page)) + rng.randrange(0, 4)
    win = CacheSpec("window", (1, 16), window=window)
    cache = CacheManager([CacheNeed(FULL, None, None), CacheNeed(win, None, None)], page, [200, win_pages], conc,
                         torch.float32, "cpu", allocate=False)
    sched = Scheduler(cache, conc, budget, chunk, 120, (3,))
    seqs = [Sequence(i, [rng.randrange(10) for _ in range(rng.randrange(1, 80))], rng.randrange(1, 30))
            for i in range(20)]
    sched.add_sequences(seqs)
    run(cache, sched, token_of=lambda s: rng.randrange(10))
    assert len(sched.completed) == 20 and not sched.running and not sched.waiting_queue
    for s in sched.completed:
        assert s.status is Status.COMPLETE and s.finish_reason in ("eos", "length", "context"), \
            (s.seq_id, s.status, s.finish_reason, page, window, win_pages, chunk, budget)
    assert cache.groups[1].pool.high_water <= win_pages
    assert all(g.pool.num_free == g.pool.num_pages for g in cache.groups)
    cache.check_invariants()


@pytest.mark.parametrize("seed", range(4))
def test_groups_with_different_page_sizes_under_pressure(seed):
    """Two groups whose pages hold 4 and 3 tokens, pools of different sizes: every plan fits both pools, requests
    wait or are preempted for pages of either group, and all of them finish with the books clean."""
    rng = random.Random(seed)
    needs = [CacheNeed(FULL, None, None), CacheNeed(CacheSpec("full", (8,), tensors=1, page_size=3), None, None)]
    cache = CacheManager(needs, 4, [rng.randrange(8, 14), rng.randrange(10, 18)], 4, torch.float32, "cpu", allocate=False)
    sched = Scheduler(cache, 4, 12, 6, 1000, (), False)
    seqs = [Sequence(i, [1] * rng.randrange(1, 24), rng.randrange(1, 9)) for i in range(20)]
    sched.add_sequences(seqs)
    tight = [0, 0]
    while not sched.is_done():
        work = sched.plan()
        assert work, "unfinished requests, no work"
        free = cache.free_pages()
        sched.process_results(work, fake_step(cache, work))
        for g in range(2):
            tight[g] += cache.groups[g].pool.num_free == 0 or free[g] == 0
    assert len(sched.completed) == 20
    for s in sched.completed:
        if s.status is Status.COMPLETE and s.finish_reason == "length":
            assert len(s.output_ids) == s.max_new_tokens
        else:
            needs_pages = cache.peak_pages(s.prompt_len + 1, 1)
            assert s.status is Status.FAILED or s.finish_reason == "cache"
            assert any(n > g.pool.num_pages for n, g in zip(needs_pages, cache.groups)) or s.finish_reason == "cache"
    assert cache.free_pages() == [g.pool.num_pages for g in cache.groups]
    cache.check_invariants()
