"""The cache manager on the host: no page lost, held twice or freed twice, under random orders."""

import random

import numpy as np
import pytest
import torch

from freetoken_b200.cache import CacheManager, PagePool, StateSlotPool
from freetoken_b200.config.spec import PagedKVNeed, StateNeed
from freetoken_b200.errors import CacheError

CPU = torch.device("cpu")
FULL = PagedKVNeed((("k", 2, 16), ("v", 2, 16)))
WIN = PagedKVNeed((("k", 2, 16), ("v", 2, 16)), window=10)
STATE = StateNeed((("s", (3, 4), "float32"),))


def make(needs, pages=12, page=4, reqs=4, seq=64):
    return CacheManager(needs, page, pages, reqs, seq, torch.float32, CPU, poison=True, max_step_tokens=seq)


def test_page_pool_basics():
    p = PagePool(3)
    a = p.alloc(2)
    assert 0 not in a and p.free_count == 1
    with pytest.raises(CacheError, match="out of pages"):
        p.alloc(2)
    p.free(a[:1])
    with pytest.raises(CacheError, match="freed twice"):
        p.free(a[:1])
    assert p.alloc(1) == a[:1]  # last freed, first reused
    with pytest.raises(CacheError):
        p.free([0])
    s = StateSlotPool(2)
    x, y = s.alloc(), s.alloc()
    with pytest.raises(CacheError):
        s.alloc()
    s.free(x)
    with pytest.raises(CacheError):
        s.free(x)
    assert s.alloc() == x and y != x


def test_groups_by_need():
    m = make([(0, FULL), (1, WIN), (2, FULL), (3, STATE), (5, WIN)])
    assert len(m.paged) == 2 and len(m.state) == 1
    assert m.paged[0].entries == [0, 2] and m.paged[1].entries == [1, 5]
    assert m.paged[0].slabs["k"].shape == (2, 13, 2, 4, 16)
    v0, v2 = m.view(0), m.view(2)
    assert v0.slabs["k"].data_ptr() != v2.slabs["k"].data_ptr()
    assert m.view(3).tensors["s"].shape == (5, 3, 4) and m.view(4) is None
    assert m.paged[1].pool.num_pages <= 12  # a windowed group has pages of its own
    assert CacheManager.bytes_per_token([(0, FULL), (1, WIN), (3, STATE)], 2) == 2 * 64 * 2


def test_slots_follow_the_block_table():
    m = make([(0, FULL)])
    m.open("a")
    plan = m.begin_step([("a", 6)])
    row = plan.rows[0]
    pages = m.paged[0].table_host[row, :2]
    assert list(plan.slot_maps[0]) == [pages[0] * 4 + i for i in range(4)] + [pages[1] * 4, pages[1] * 4 + 1]
    ups = m.take_updates(0)
    assert ups == [(row * m.width + 0, int(pages[0])), (row * m.width + 1, int(pages[1]))]
    m.end_step()
    plan = m.begin_step([("a", 3)])
    assert plan.kv_lens == [9] and not plan.fresh[0]
    assert list(plan.slot_maps[0][:2]) == [pages[1] * 4 + 2, pages[1] * 4 + 3]
    m.end_step()
    m.check()
    m.close("a")
    m.check()
    assert m.paged[0].pool.free_count == 12


def test_out_of_pages_takes_nothing():
    m = make([(0, FULL)], pages=3)
    m.open("a")
    m.open("b")
    m.begin_step([("a", 8)])
    m.end_step()
    with pytest.raises(CacheError, match="out of pages"):
        m.begin_step([("a", 1), ("b", 5)])
    m.check()
    assert m.length("a") == 8 and m.length("b") == 0 and m.paged[0].pool.free_count == 1
    m.begin_step([("b", 4)])
    m.abort_step()  # a step that did not run gives its pages back
    m.check()
    assert m.paged[0].pool.free_count == 1 and m.length("b") == 0
    with pytest.raises(CacheError, match="longest sequence"):
        m.begin_step([("a", 100)])
    with pytest.raises(CacheError, match="twice"):
        m.begin_step([("a", 1), ("a", 1)])
    with pytest.raises(CacheError):
        m.begin_step([("zz", 1)])


def test_window_gives_pages_back_and_reuses_them():
    m = make([(0, WIN)], pages=40, page=4, seq=400)
    m.open("a")
    pool = m.paged[0].pool
    m.begin_step([("a", 30)])  # a long portion needs all its pages during the step
    assert pool.num_pages - pool.free_count == 8
    m.end_step()
    held = pool.num_pages - pool.free_count
    assert held <= 4  # only what the next query (position 30, window 10) can still read
    for _ in range(200):
        m.begin_step([("a", 1)])
        m.end_step()
        m.check()
        assert pool.num_pages - pool.free_count <= 4
    assert pool.handed_out > pool.num_pages  # pages went round more than once
    first = m.paged[0].first_live[m.requests["a"].row]
    assert first == (230 - 10 + 1) // 4
    m.close("a")
    m.check()


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_keep_every_page_accounted_for(seed):
    rng = random.Random(seed)
    needs = [(0, FULL), (1, WIN), (2, STATE), (3, FULL)]
    m = make(needs, pages=20, page=4, reqs=4, seq=48)
    live, next_id = {}, 0
    for _ in range(300):
        action = rng.random()
        if action < 0.25 and len(live) < 4:
            m.open(next_id)
            live[next_id] = 0
            next_id += 1
        elif action < 0.4 and live:
            rid = rng.choice(list(live))
            m.close(rid)
            del live[rid]
        elif live:
            picks = rng.sample(list(live), rng.randint(1, len(live)))
            entries = [(r, rng.choice([1, 1, 1, 2, 5, 9])) for r in picks if live[r] < 40]
            entries = [(r, min(n, 48 - live[r])) for r, n in entries]
            if not entries:
                continue
            try:
                plan = m.begin_step(entries)
            except CacheError as e:
                assert "out of pages" in str(e)
                m.check()
                continue
            for g in m.paged:  # no slot is given to two tokens of one step
                s = plan.slot_maps[g.index]
                s = s[s >= 0]
                assert len(set(s.tolist())) == len(s)
            if rng.random() < 0.1:
                m.abort_step()
            else:
                m.end_step()
                for r, n in entries:
                    live[r] += n
        m.check()
        for r, n in live.items():
            assert m.length(r) == n
    for rid in list(live):
        m.close(rid)
    m.check()
    assert all(g.pool.free_count == g.pool.num_pages for g in m.paged)
    assert m.slots.free_count == 4 and m.free_request_slots() == 4


def test_close_is_refused_during_a_step_and_state_slots_are_fresh_once():
    m = make([(0, FULL), (1, STATE)])
    m.open("a")
    plan = m.begin_step([("a", 2)])
    assert plan.fresh == [True] and plan.state_slots[0] >= 1
    with pytest.raises(CacheError, match="in flight"):
        m.close("a")
    m.end_step()
    assert m.begin_step([("a", 1)]).fresh == [False]
    m.end_step()
    with pytest.raises(CacheError):
        m.open("a")
    for r in "bcd":
        m.open(r)
    with pytest.raises(CacheError, match="no request slot"):
        m.open("e")


@pytest.mark.parametrize("seed", range(8))
def test_admission_reserves_what_a_windowed_request_holds_at_its_peak(seed):
    """``pages_to_admit`` is a bound on what a request ever holds while a step runs, for full and
    windowed groups, whatever the portions are; and it is reached (the bound is not loose by more
    than a page for the windowed group)."""
    rng = random.Random(seed)
    page = rng.choice([2, 4, 8])
    window = rng.choice([1, 3, 8, 10, 17])
    step = rng.choice([1, 2, 5, 16, 64])
    total = rng.randint(1, 200)
    need = PagedKVNeed((("k", 1, 16), ("v", 1, 16)), window=window)
    m = CacheManager([(0, FULL), (1, need)], page, 200, 2, 256, torch.float32, CPU, max_step_tokens=step)
    bound = m.pages_to_admit(total)
    assert bound[0] == -(-total // page)
    m.open("a")
    peak, fed = [0, 0], 0
    while fed < total:
        n = min(step if rng.random() < 0.5 else rng.randint(1, step), total - fed)
        m.begin_step([("a", n)])
        for i, g in enumerate(m.paged):
            peak[i] = max(peak[i], g.pool.num_pages - g.pool.free_count)
        m.end_step()
        fed += n
    assert peak[0] == bound[0]
    assert peak[1] <= bound[1], (page, window, step, total, peak, bound)
    # with whole steps every time the bound is tight within one page
    m.close("a")
    m.open("b")
    peak_b, fed = 0, 0
    while fed < total:
        n = min(step, total - fed)
        m.begin_step([("b", n)])
        peak_b = max(peak_b, m.paged[1].pool.num_pages - m.paged[1].pool.free_count)
        m.end_step()
        fed += n
    assert bound[1] - peak_b <= 2
    assert m.pages_to_admit(total, step_tokens=1)[1] <= bound[1]
