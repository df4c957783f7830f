"""The cache manager without a device: no page is lost, held twice or freed twice, under random
orders of requests; windowed groups give pages back; state slots are reused."""
import numpy as np
import pytest

from inference_bench_b200.cache.manager import CacheError, CacheManager, OutOfPages
from inference_bench_b200.cache.pages import PagePool, PagePoolError
from inference_bench_b200.parts.base import FixedState, PagedKV


def test_page_pool_basics():
    pool = PagePool(3)
    a, b, c = pool.allocate(), pool.allocate(), pool.allocate()
    assert sorted([a, b, c]) == [0, 1, 2] and pool.allocate() is None and pool.free_pages == 0
    pool.release(b)
    assert pool.allocate() == b          # the page just freed is handed out first
    pool.share(a)
    pool.release(a)
    assert pool.refcount(a) == 1 and pool.free_pages == 0
    pool.release(a)
    with pytest.raises(PagePoolError, match="nobody holds"):
        pool.release(a)
    with pytest.raises(PagePoolError):
        pool.share(a)
    with pytest.raises(PagePoolError, match="outside"):
        pool.release(7)
    pool.check()


def _manager(window=None, pages=12, page=4, slots=3, limit=64):
    needs = [PagedKV(2, 8, None), PagedKV(2, 8, window), PagedKV(2, 8, None), FixedState((5,)), None]
    return CacheManager(needs, page, pages, slots, limit, sources=[0, 1, 2, 3, 2])


def test_groups_by_need():
    m = _manager(window=6)
    assert len(m.groups) == 2                                     # full attention, and the windowed layer
    assert m.groups[0].entries == [0, 2] and m.groups[1].entries == [1]
    assert m.place == {0: (0, 0), 1: (1, 0), 2: (0, 1)} and list(m.states) == [3]
    same = _manager(window=None)
    assert len(same.groups) == 1 and same.groups[0].entries == [0, 1, 2]


def test_extend_commit_release_and_tables():
    m = _manager()
    m.admit("a")
    m.extend("a", 9)                                               # 3 pages of 4
    assert m.used_pages() == [3] and (m.table(0, "a")[:3] >= 0).all() and m.table(0, "a")[3] == -1
    m.extend("a", 9)                                               # asking again takes nothing more
    assert m.used_pages() == [3]
    m.commit("a", 9)
    assert m.length("a") == 9 and m.pages_missing("a", 12) == [0] and m.pages_missing("a", 13) == [1]
    m.check()
    m.release("a")
    assert m.used_pages() == [0] and m.free_slots() == 3
    with pytest.raises(CacheError):
        m.length("a")
    m.check()


def test_extend_is_all_or_nothing_and_rolls_back():
    m = _manager(window=100, pages=4)                              # two groups of 4 pages
    m.admit("a")
    m.admit("b")
    m.extend("a", 12)
    m.commit("a", 12)
    with pytest.raises(OutOfPages):
        m.extend("b", 8)                                           # needs 2 pages per group, 1 is free
    assert m.used_pages() == [3, 3] and (m.table(0, "b") == -1).all()
    m.extend("b", 4)
    m.shrink_to_committed("b")                                     # an extend that no commit followed
    assert m.used_pages() == [3, 3]
    with pytest.raises(OutOfPages, match="limit"):
        m.extend("a", 65)
    m.check()


def test_window_gives_pages_back_and_they_are_reused():
    m = _manager(window=6, pages=10, page=4)
    m.admit("a")
    held = []
    for length in range(1, 41):
        m.extend("a", length)
        m.commit("a", length)
        m.check()
        held.append(m.used_pages()[1])
        # every key the next token may see is still there: positions length-6+1 .. length-1
        first_needed = max(0, length - 6 + 1)
        assert (m.table(1, "a")[first_needed // 4: -(-length // 4)] >= 0).all()
        assert (m.table(1, "a")[:first_needed // 4] == -1).all()
    assert max(held) <= 3                       # a window of 6 tokens never holds more than 3 pages of 4
    assert m.used_pages()[0] == 10              # the full-attention group keeps all 40 positions
    m.release("a")
    assert m.used_pages() == [0, 0]


def test_window_full_group_runs_out_but_window_group_does_not():
    m = _manager(window=6, pages=6, page=4)
    m.admit("a")
    with pytest.raises(OutOfPages):
        for length in range(1, 41):
            m.extend("a", length)
            m.commit("a", length)
    assert m.length("a") == 24                                     # 6 pages of 4 in the full-attention group
    m.check()


def test_slots_and_fixed_state_bookkeeping():
    m = _manager(slots=2)
    s0, s1 = m.admit("a"), m.admit("b")
    assert {s0, s1} == {0, 1} and m.scratch_slot == 2
    with pytest.raises(CacheError, match="no free slot"):
        m.admit("c")
    with pytest.raises(CacheError, match="already"):
        m.admit("a")
    m.release("a")
    assert m.admit("c") == s0
    m.check()


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_keep_the_invariants(seed):
    rng = np.random.default_rng(seed)
    m = _manager(window=int(rng.integers(3, 20)), pages=int(rng.integers(6, 20)), page=int(rng.choice([2, 4, 8])), slots=4, limit=80)
    live: dict[int, int] = {}
    next_id = 0
    for _ in range(1500):
        op = rng.random()
        if op < 0.15 and m.free_slots():
            m.admit(next_id)
            live[next_id] = 0
            next_id += 1
        elif op < 0.8 and live:
            r = int(rng.choice(list(live)))
            new = live[r] + int(rng.integers(1, 12))
            fits = m.can_extend(r, new)
            try:
                m.extend(r, new)
                assert fits
                if rng.random() < 0.9:
                    m.commit(r, new)
                    live[r] = new
                else:
                    m.shrink_to_committed(r)
            except OutOfPages:
                assert not fits or new > 80
        elif live:
            r = int(rng.choice(list(live)))
            m.release(r)
            del live[r]
        m.check()
        for r, n in live.items():
            assert m.length(r) == n
    for r in list(live):
        m.release(r)
    m.check()
    assert m.used_pages() == [0] * len(m.groups) and m.free_slots() == 4
