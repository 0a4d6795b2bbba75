"""The cache manager's bookkeeping (no GPU): no page lost, held twice or freed twice, under
random orders of requests; windows give pages back; a failed reservation changes nothing."""
import random

import pytest

from air_b200.cache.manager import CacheError, CacheManager, OutOfPages, PagePool
from air_b200.parts.base import PagedKV, SlotState

FULL = PagedKV(2, 16, None)
WIN = PagedKV(2, 16, 40)


def manager(needs, pages=8, page=16, slots=4):
    return CacheManager(needs, page, pages, slots, allocate=False)


def test_pool_refuses_double_free_and_foreign_free():
    pool = PagePool(3)
    a, b = pool.take("x"), pool.take("y")
    pool.give(a, "x")
    with pytest.raises(CacheError, match="twice"):
        pool.give(a, "x")
    with pytest.raises(CacheError, match="belongs"):
        pool.give(b, "x")
    assert pool.take("z") == a, "the page freed last is used again first"
    pool.take("z")
    with pytest.raises(OutOfPages):
        pool.take("z")
    pool.check()


def test_groups_by_need_and_pages_of_their_own():
    m = manager([(FULL,), (WIN,), (WIN,), (), (FULL,)])
    assert len(m.groups) == 2
    assert m.groups[0].runs == [0, 4] and m.groups[1].runs == [1, 2]
    assert m.views(3) == () and m.views(1)[0].group == 1
    m.open("a")
    m.reserve([("a", 100)])
    m.commit("a", 100)
    full, win = m.sequences["a"].pages
    assert len(full) == 7 and all(p >= 0 for p in full)
    # window 40: keys below 100 - 40 + 1 = 61 are out of reach -> blocks 0..2 (tokens 0..47) are free
    assert [p >= 0 for p in win] == [False, False, False, True, True, True, True]
    assert m.groups[0].pool.used_pages == 7 and m.groups[1].pool.used_pages == 4
    m.check()
    m.close("a")
    assert m.free_pages() == 8
    m.check()


def test_failed_reservation_changes_nothing():
    m = manager([(FULL,)], pages=5)
    m.open("a"); m.open("b")
    m.reserve([("a", 30)])
    m.commit("a", 30)
    before = (list(m.sequences["a"].pages[0]), m.free_pages())
    with pytest.raises(OutOfPages):
        m.reserve([("a", 10), ("b", 50)])     # a needs 1 more page, b needs 4: only 3 are free
    assert (list(m.sequences["a"].pages[0]), m.free_pages()) == before and m.sequences["b"].pages[0] == []
    m.check()
    m.reserve([("a", 10), ("b", 30)])
    m.check()


def test_trim_gives_back_uncommitted_pages():
    m = manager([(FULL,)])
    m.open("a")
    m.reserve([("a", 20)])
    m.commit("a", 20)
    m.reserve([("a", 60)])
    assert m.used_pages("a") == 5
    m.trim("a")
    assert m.used_pages("a") == 2 and m.length("a") == 20
    m.check()


def test_slots_are_reused_and_limited():
    m = manager([(SlotState((4,)),)], slots=2)
    a, b = m.open("a").slot, m.open("b").slot
    assert {a, b} == {0, 1}
    with pytest.raises(CacheError, match="slots"):
        m.open("c")
    m.close("a")
    assert m.open("c").slot == a
    with pytest.raises(CacheError):
        m.open("c")
    with pytest.raises(CacheError):
        m.close("zzz")
    m.check()


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_keep_the_books(seed):
    rng = random.Random(seed)
    m = manager([(FULL,), (WIN,), (SlotState((2,)),)], pages=24, slots=5)
    live, counter = {}, 0
    for _ in range(600):
        action = rng.random()
        if action < 0.25 and len(live) < 5:
            name = f"r{counter}"; counter += 1
            m.open(name); live[name] = 0
        elif action < 0.85 and live:
            batch = [(r, rng.choice([1, 1, 1, 2, 7, 16, 33])) for r in rng.sample(sorted(live), rng.randint(1, len(live)))]
            try:
                m.reserve(batch)
            except OutOfPages:
                m.check()
                victim = rng.choice(sorted(live))
                m.close(victim); del live[victim]
            else:
                if rng.random() < 0.1:      # the step failed: nothing is committed
                    for r, _ in batch:
                        m.trim(r)
                else:
                    for r, n in batch:
                        m.commit(r, n); live[r] += n
        elif live:
            victim = rng.choice(sorted(live))
            m.close(victim); del live[victim]
        m.check()
        for r, n in live.items():
            assert m.length(r) == n
            full, win = m.sequences[r].pages
            assert sum(p >= 0 for p in full) == -(-n // 16) or len(full) >= -(-n // 16)
            first_needed = max(0, n - 40 + 1) // 16
            assert all(p >= 0 for p in win[first_needed:-(-n // 16)]), "every key inside the window has its page"
    for r in list(live):
        m.close(r)
    m.check()
    assert all(g.pool.free_pages == 24 for g in m.groups)
    assert any(g.pool.takes > 24 for g in m.groups)
