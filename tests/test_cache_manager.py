"""Cache manager bookkeeping on the host: no page lost, held twice or freed twice,
under random orders of requests; windows give pages back; state slots."""
import random

import pytest
import torch

from batchspec_b200.cache import CacheManager, OutOfPages, PagePool, StateSlots
from batchspec_b200.models.decoder import CacheNeed
from batchspec_b200.parts import CacheSpec, StateSpec

FULL = CacheSpec("full", (2, 16))
WIN = CacheSpec("window", (2, 16), window=10)


def manager(needs, page_size=4, num_pages=12, max_requests=4):
    return CacheManager(needs, page_size, num_pages, max_requests, torch.float32, "cpu", allocate=False)


def test_pool_hands_out_each_page_once_and_takes_it_back_once():
    pool = PagePool(5)
    a = pool.allocate(3)
    b = pool.allocate(2)
    assert sorted(a + b) == [0, 1, 2, 3, 4] and pool.num_free == 0
    with pytest.raises(OutOfPages):
        pool.allocate(1)
    pool.free(a)
    with pytest.raises(RuntimeError, match="not held"):
        pool.free([a[0]])
    with pytest.raises(RuntimeError, match="not held"):
        pool.free([99])
    c = pool.allocate(3)
    assert sorted(c) == sorted(a), "freed pages are handed out again"
    assert pool.high_water == 5


def test_state_slots():
    s = StateSlots(2)
    x, y = s.take(), s.take()
    assert {x, y} == {0, 1}
    with pytest.raises(OutOfPages):
        s.take()
    s.give(x)
    with pytest.raises(RuntimeError):
        s.give(x)
    assert s.take() == x


def test_groups_follow_the_needs():
    needs = [CacheNeed(FULL, None, None), CacheNeed(WIN, None, None), CacheNeed(FULL, None, None),
             CacheNeed(FULL, None, 0), CacheNeed(None, StateSpec((3,)), None)]
    m = CacheManager(needs, 4, 6, 3, torch.float32, "cpu")
    assert len(m.groups) == 2 and m.groups[0].runs == [0, 2] and m.groups[1].runs == [1]
    assert m.groups[0].pages.shape == (2, 6, 2, 4 * 32)
    lc = m.layer_caches
    assert lc[0].group == 0 and lc[1].group == 1 and lc[2].group == 0
    assert lc[3].kv.data_ptr() == lc[0].kv.data_ptr() and not lc[3].owner and lc[0].owner
    assert lc[4].kv is None and lc[4].state.shape == (3, 3)


def test_reserve_commit_release_and_page_arithmetic():
    m = manager([CacheNeed(FULL, None, None)])
    m.admit("a")
    assert m.pages_needed(0, 1) == [1] and m.pages_needed(3, 1) == [0] and m.pages_needed(4, 1) == [1]
    assert m.pages_needed(3, 6) == [2]
    m.reserve("a", 5)
    m.commit("a", 5)
    assert len(m.requests["a"].tables[0]) == 2 and m.length("a") == 5
    m.reserve("a", 3)                     # 5 -> 8: still two pages
    m.commit("a", 3)
    assert len(m.requests["a"].tables[0]) == 2
    m.admit("b")
    with pytest.raises(OutOfPages):
        m.reserve("b", 4 * 11)            # all or nothing
    assert m.requests["b"].tables[0] == [] and m.groups[0].pool.num_free == 10
    assert m.can_reserve([(8, 1), (0, 36)]) and not m.can_reserve([(8, 1), (0, 37)])
    m.check_invariants()
    m.release("a")
    with pytest.raises(KeyError):
        m.release("a")
    m.release("b")
    assert m.groups[0].pool.num_free == 12
    m.check_invariants()


def test_window_gives_back_pages_it_has_passed():
    m = manager([CacheNeed(FULL, None, None), CacheNeed(WIN, None, None)], page_size=4, num_pages=16)
    m.admit("a")
    m.reserve("a", 23)
    m.commit("a", 23)
    full, win = m.requests["a"].tables
    assert all(p >= 0 for p in full) and len(full) == 6
    # next query at position 23 reads keys 14..23: pages 0..2 (positions 0..11) are dead
    assert win[:3] == [-1, -1, -1] and all(p >= 0 for p in win[3:]) and len(win) == 6
    assert m.groups[1].pool.num_held == 3 and m.groups[0].pool.num_held == 6
    for _ in range(9):
        m.reserve("a", 1)
        m.commit("a", 1)
    assert m.groups[1].pool.num_held <= 4          # stays bounded by the window
    m.check_invariants()
    m.release("a")
    assert m.groups[1].pool.num_held == 0 == m.groups[0].pool.num_held


def test_state_is_zeroed_at_admission():
    m = CacheManager([CacheNeed(None, StateSpec((2, 2)), None)], 4, 1, 2, torch.float32, "cpu")
    rc = m.admit("a")
    m.state_tensors[0][rc.slot] += 5
    m.release("a")
    rc2 = m.admit("b")
    assert rc2.slot == rc.slot and float(m.state_tensors[0][rc2.slot].abs().sum()) == 0


def test_groups_with_pages_of_their_own_size_and_one_tensor_per_token():
    """A mixer may store one tensor per token and choose its group's page size: the same request then has block
    tables of different lengths, and every count of pages is per group."""
    latent = CacheSpec("full", (12,), tensors=1, page_size=3)
    m = CacheManager([CacheNeed(FULL, None, None), CacheNeed(latent, None, None), CacheNeed(FULL, None, None)],
                     4, 6, 2, torch.float32, "cpu", scratch_page=True)
    assert [g.page_size for g in m.groups] == [4, 3] and [g.runs for g in m.groups] == [[0, 2], [1]]
    assert [g.pool.num_pages for g in m.groups] == [6, 8], "the same number of tokens in pages of either size"
    assert m.groups[0].pages.shape == (2, 7, 2, 4 * 32) and m.groups[1].pages.shape == (1, 9, 1, 3 * 12)
    assert m.layer_caches[1].kv.shape == (9, 1, 36)
    m.admit("a")
    assert m.pages_needed(0, 7) == [2, 3] and m.pages_missing("a", 7) == [2, 3]
    m.reserve("a", 7)
    m.commit("a", 7)
    assert [len(t) for t in m.requests["a"].tables] == [2, 3]
    assert m.pages_missing("a", 1) == [0, 0] and m.pages_missing("a", 2) == [1, 0] and m.pages_missing("a", 3) == [1, 1]
    assert m.room_for(7, [1, 0]) == 2 and m.room_for(7, [0, 5]) == 1 and m.room_for(7, [2, 2]) == 8
    assert m.peak_pages(10, 10) == [3, 4]
    m.admit("b")
    assert m.free_pages() == [4, 5]
    assert m.can_reserve([(0, 15)]) and not m.can_reserve([(0, 15), (7, 2)])         # group 0: 4 + 1 > 4 free
    assert not m.can_reserve([(0, 16)])                                              # group 1: 6 > 5 free
    with pytest.raises(OutOfPages):
        m.reserve("b", 16)                                                           # group 0 alone would have room
    assert m.requests["b"].tables == [[], []], "all or nothing, over all groups"
    m.check_invariants()
    m.release_all()
    assert m.free_pages() == [6, 8] and m.scratch_pages() == [6, 8] and m.scratch_slot() == 2


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_keep_the_books(seed):
    rng = random.Random(seed)
    needs = [CacheNeed(FULL, None, None), CacheNeed(WIN, None, None),
             CacheNeed(CacheSpec("full", (5,), tensors=1, page_size=rng.choice([3, 16])), None, None),
             CacheNeed(CacheSpec("window", (2, 8), window=7, page_size=2), None, None)]
    m = manager(needs, page_size=rng.choice([1, 4, 8]), num_pages=rng.randrange(6, 30), max_requests=5)
    live, next_id, refused = [], 0, 0
    for _ in range(600):
        op = rng.random()
        if op < 0.25 and len(live) < 5:
            m.admit(next_id)
            live.append(next_id)
            next_id += 1
        elif op < 0.85 and live:
            rid = rng.choice(live)
            n = rng.choice([1, 1, 1, 2, 5, 9, 17])
            before = [list(t) for t in m.requests[rid].tables]
            try:
                m.reserve(rid, n)
            except OutOfPages:
                refused += 1
                assert [list(t) for t in m.requests[rid].tables] == before
            else:
                m.commit(rid, n)
        elif live:
            rid = live.pop(rng.randrange(len(live)))
            m.release(rid)
        m.check_invariants()
    assert refused > 0, "the pool was never under pressure"
    m.release_all()
    m.check_invariants()
    assert all(g.pool.num_free == g.pool.num_pages for g in m.groups)


def test_peak_pages_bound_what_a_request_ever_holds():
    """``peak_pages`` is what the scheduler compares with the pools' sizes: never less than what a request holds
    in any group at any moment, whatever the window, the page size and the portions; and small for a window."""
    rng = random.Random(3)
    for _ in range(200):
        ps, window = rng.choice([1, 4, 8, 16]), rng.randint(1, 40)
        portion, total = rng.randint(1, 30), rng.randint(1, 200)
        needs = [CacheNeed(FULL, None, None), CacheNeed(CacheSpec("window", (2, 16), window=window), None, None)]
        m = CacheManager(needs, ps, 400, 1, torch.float32, "cpu", allocate=False)
        peak = m.peak_pages(total, portion)
        assert peak[0] == -(-total // ps) and peak[1] <= peak[0]
        assert peak[1] <= (window + portion) // ps + 3
        m.admit("r")
        done, worst = 0, [0, 0]
        while done < total:
            n = min(rng.randint(1, portion), total - done)
            m.reserve("r", n)
            worst = [max(w, g.pool.num_held) for w, g in zip(worst, m.groups)]
            m.commit("r", n)
            done += n
        assert worst[0] <= peak[0] and worst[1] <= peak[1], (ps, window, portion, total, worst, peak)
