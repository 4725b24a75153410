"""The cache manager on the host: no page lost, held twice or freed twice, under random
orders of requests; windows give pages back; state slots are handed out and zeroed."""

import random

import pytest
import torch

from ninfer_amd_mi50_b200.cache import CacheManager, OutOfPages, OutOfSlots, PagePool
from ninfer_amd_mi50_b200.parts.base import CacheSpec, StateSpec

FULL = CacheSpec("full", 2, 16)
WIN = CacheSpec("window", 2, 16, 40)


def manager(specs=(FULL, FULL), states=(None, None), pages=8, reqs=3, page=16, ctx=256, allocate=False):
    return CacheManager(list(specs), list(states), page_size=page, num_pages=pages, max_requests=reqs,
                        max_context=ctx, allocate=allocate)


def test_pool_take_and_give_back():
    p = PagePool(4)
    a = p.take(3)
    assert sorted(a) == [0, 1, 2] and p.num_free == 1
    with pytest.raises(OutOfPages):
        p.take(2)
    assert p.num_free == 1                     # a refused request takes nothing
    p.give_back([a[1]])
    assert p.take(1) == [a[1]]                 # the page just freed is the next one used
    with pytest.raises(AssertionError, match="freed twice"):
        p.give_back([3])
    p.give_back(a)
    with pytest.raises(AssertionError, match="freed twice"):
        p.give_back([a[0]])
    p.check()


def test_reserve_commit_close():
    m = manager()
    m.open("a")
    assert m.pages_needed("a", 17) == [2]
    m.reserve("a", 17)
    m.commit("a", 17)
    assert m.length("a") == 17 and len(m.block_table(0, "a")) == 2
    m.reserve("a", 18)                         # same page: nothing more taken
    assert m.pages_free() == [6]
    m.reserve("a", 33)
    assert m.pages_free() == [5]
    m.truncate("a")                            # the step did not run: back to 2 pages
    assert m.pages_free() == [6] and len(m.block_table(0, "a")) == 2
    with pytest.raises(AssertionError):
        m.commit("a", 40)
    m.close("a")
    assert m.pages_free() == [8]
    m.check()


def test_reserve_is_all_or_nothing_across_groups():
    m = manager(specs=(FULL, WIN), pages=4)
    m.open("a")
    m.open("b")
    m.reserve("a", 48)                          # 3 pages in each group
    m.groups[1].pool.take(1)                    # group 1 now has no page left, group 0 has one
    with pytest.raises(OutOfPages):
        m.reserve("b", 10)
    assert m.pages_free() == [1, 0] and m.block_table(0, "b") == []
    with pytest.raises(OutOfPages, match="max_context"):
        m.reserve("a", 10_000)


def test_window_group_releases_pages_the_window_has_passed():
    m = manager(specs=(FULL, WIN), pages=16)
    m.open("a")
    n = 0
    for step in [30, 1, 1, 50, 1, 1, 1, 60]:
        n += step
        m.reserve("a", n)
        m.commit("a", n)
        full, win = m.block_table(0, "a"), m.block_table(1, "a")
        assert all(p >= 0 for p in full) and len(full) == (n + 15) // 16
        first_key = max(0, n - 40 + 1)          # oldest key a later position can still see
        for lp, p in enumerate(win):
            assert (p >= 0) == ((lp + 1) * 16 > first_key), (n, lp, win)
        m.check()
    assert m.pages_free()[1] > m.pages_free()[0]
    m.close("a")
    assert m.pages_free() == [16, 16]


def test_state_slots():
    m = manager(states=(None, StateSpec((3, 4))), reqs=2, allocate=True)
    s = m.open("a")
    m.state_of(1)[s] += 5
    t = m.open("b")
    assert {s, t} == {0, 1} and m.state_of(0) is None
    with pytest.raises(OutOfSlots):
        m.open("c")
    with pytest.raises(KeyError):
        m.open("a")
    m.close("a")
    assert m.open("c") == s and float(m.state_of(1)[s].abs().sum()) == 0.0   # reused and zeroed
    m.check()


def test_bytes_per_token():
    m = manager(specs=(FULL, FULL, None, WIN), states=(None,) * 4, allocate=True)
    assert m.bytes_per_token() == 3 * 2 * 2 * 16 * 4
    assert m.total_bytes() == 2 * (2 * 9 * 2 * 2 * 16 * 16 * 4) // 2 + 9 * 2 * 2 * 16 * 16 * 4


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_lose_no_page(seed):
    rng = random.Random(seed)
    m = manager(specs=(FULL, WIN, FULL), states=(None, None, None), pages=10, reqs=4)
    live, counter = {}, 0
    for _ in range(400):
        op = rng.random()
        if op < 0.25 and len(live) < 4:
            counter += 1
            m.open(counter)
            live[counter] = 0
        elif op < 0.8 and live:
            r = rng.choice(list(live))
            new = live[r] + rng.choice([1, 1, 1, 2, 7, 16, 33])
            if m.can_reserve(r, new):
                m.reserve(r, new)
                if rng.random() < 0.9:
                    m.commit(r, new)
                    live[r] = new
                else:
                    m.truncate(r)
            else:
                free = m.pages_free()
                with pytest.raises(OutOfPages):
                    m.reserve(r, new)
                assert m.pages_free() == free
        elif live:
            r = rng.choice(list(live))
            m.close(r)
            del live[r]
        m.check()
        for r, n in live.items():
            assert m.length(r) == n
    for r in list(live):
        m.close(r)
    m.check()
    assert m.pages_free() == [10, 10]


def test_a_partly_covered_page_is_cleared_when_it_is_handed_out_again():
    """A page that goes to a second owner and is not covered to its last row by the reservation
    is zeroed first (what lies beyond the new owner's position in it is multiplied by zero
    probabilities, and must be finite).  Pages covered completely are overwritten by the step
    before anything reads them, and a page handed out for the first time still has the zeros it
    was made with: both are left alone."""
    import torch
    from ninfer_amd_mi50_b200.cache.manager import CacheManager
    from ninfer_amd_mi50_b200.parts.base import CacheSpec
    spec = CacheSpec("full", 2, 8)
    cm = CacheManager([spec, spec], [None, None], page_size=4, num_pages=6, max_requests=2, max_context=24)
    (g,) = cm.groups
    cm.open("a")
    cm.reserve("a", 9)                       # three pages, first use: nothing to clear
    assert cm.pages_cleared == 0
    held = list(cm.block_table(0, "a"))
    g.pages[:, held] = float("nan")          # whatever "a" left there
    cm.commit("a", 9)
    cm.close("a")
    cm.open("b")
    cm.reserve("b", 6)                       # two of "a"'s pages again: rows 0-3 and 4-5 (+ two stale rows)
    t = cm.block_table(0, "b")
    assert set(t) <= set(held) and cm.pages_cleared == 1
    assert bool(torch.isnan(g.pages[:, t[0]]).all())                   # covered whole: the step overwrites it
    assert float(g.pages[:, t[1]].abs().sum()) == 0.0                 # covered in part: zeroed
    cm.commit("b", 6)
    cm.reserve("b", 8)                       # same page, further rows: it is not taken again
    cm.reserve("b", 9)                       # the third of "a"'s pages, one row of four
    assert cm.pages_cleared == 2 and float(g.pages[:, cm.block_table(0, "b")[2]].abs().sum()) == 0.0
    off = CacheManager([spec], [None], page_size=4, num_pages=2, max_requests=1, max_context=8, clear_reused_pages=False)
    off.open("a"); off.reserve("a", 8); off.groups[0].pages[:, :2] = 1.0; off.commit("a", 8); off.close("a")
    off.open("b"); off.reserve("b", 7)
    assert off.pages_cleared == 0 and float(off.groups[0].pages[:, :2].sum()) > 0
