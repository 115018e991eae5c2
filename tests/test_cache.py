"""The cache manager on the host: no page lost, held twice or freed twice,
under random orders of requests; windows give pages back; slots (no GPU)."""
import random
from types import SimpleNamespace

import pytest

from infernum_b200.cache import CacheManager, PagePool
from infernum_b200.errors import CacheError, OutOfPagesError
from infernum_b200.parts.base import PagedCacheSpec, StateSpec


def need(pos, paged=None, state=None, cache_of=None):
    return SimpleNamespace(position=pos, paged=paged, state=state, cache_of=cache_of)


FULL = PagedCacheSpec(2, 16, 0)
WIN = PagedCacheSpec(2, 16, 10)


def test_pool_lifo_and_errors():
    pool = PagePool(4)
    a, b = pool.allocate(), pool.allocate()
    assert (a, b) == (0, 1) and pool.num_free == 2
    pool.free(a)
    assert pool.allocate() == a  # a returned page is used again first
    assert pool.reuses == 1
    with pytest.raises(CacheError, match="twice"):
        pool.free(3)
    with pytest.raises(CacheError, match="belong"):
        pool.free(9)
    pool.allocate_many(2)
    with pytest.raises(OutOfPagesError):
        pool.allocate()
    with pytest.raises(OutOfPagesError):
        pool.allocate_many(1)


def test_allocate_many_is_all_or_nothing():
    pool = PagePool(3)
    pool.allocate()
    with pytest.raises(OutOfPagesError):
        pool.allocate_many(3)
    assert pool.num_free == 2


def test_groups_by_need_and_shared_caches():
    cm = CacheManager([need(0, FULL), need(1, WIN), need(2, FULL), need(3, cache_of=1),
                       need(4, None, StateSpec((3,)))], page_size=4, num_pages=8, max_requests=2)
    assert len(cm.groups) == 2
    assert cm.groups[0].positions == [0, 2] and cm.groups[1].positions == [1]
    lc = cm.layer_caches
    assert lc[0].group == 0 and lc[2].group == 0 and lc[1].group == 1
    assert lc[3].group == 1 and lc[3].owner is False and lc[0].owner is True
    assert lc[4].group == -1


def test_extend_commit_release():
    cm = CacheManager([need(0, FULL)], page_size=4, num_pages=5, max_requests=2)
    a = cm.admit("a")
    cm.extend(a, 6)
    assert a.tables[0] == [0, 1] and a.reserved_tokens == 6 and a.num_tokens == 0
    cm.commit(a, 6)
    cm.extend(a, 2)  # fits the second page
    assert a.tables[0] == [0, 1]
    cm.extend(a, 1)
    assert a.tables[0] == [0, 1, 2]
    with pytest.raises(CacheError, match="more tokens"):
        cm.commit(a, 4)
    b = cm.admit("b")
    with pytest.raises(OutOfPagesError):
        cm.extend(b, 9)
    assert b.tables[0] == [] and cm.free_pages() == [2]  # nothing was taken
    cm.cancel_reservation(a)
    assert a.tables[0] == [0, 1] and a.reserved_tokens == 6
    cm.release(a)
    with pytest.raises(CacheError):
        cm.release(a)
    with pytest.raises(CacheError):
        cm.extend(a, 1)
    cm.extend(b, 9)
    assert sorted(b.tables[0]) == [0, 1, 2]
    cm.check_invariants()


def test_window_gives_pages_back():
    cm = CacheManager([need(0, WIN), need(1, FULL)], page_size=4, num_pages=16, max_requests=1)
    r = cm.admit("r")
    for _ in range(10):
        cm.extend(r, 3)
        cm.commit(r, 3)
        cm.check_invariants()
        win, full = r.tables
        n = r.num_tokens
        first_needed = n - 10 + 1
        for i, page in enumerate(win):
            if (i + 1) * 4 <= first_needed:
                assert page == -1
            else:
                assert page >= 0
        assert all(p >= 0 for p in full) and len(full) == len(win) == cm.pages_for(n)
    assert cm.groups[0].pool.num_used <= 4  # at most window/page_size + 2 pages live
    cm.release(r)
    assert cm.free_pages() == [16, 16]


def test_slots():
    cm = CacheManager([need(0, FULL)], page_size=4, num_pages=4, max_requests=2)
    a, b = cm.admit("a"), cm.admit("b")
    assert {a.slot, b.slot} == {0, 1}
    with pytest.raises(OutOfPagesError, match="slots"):
        cm.admit("c")
    with pytest.raises(CacheError, match="already"):
        cm.admit("a")
    cm.release(a)
    assert cm.admit("c").slot == a.slot
    with pytest.raises(CacheError, match="not live"):
        cm.get("a")


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_keep_the_books(seed):
    rng = random.Random(seed)
    cm = CacheManager([need(0, FULL), need(1, WIN), need(2, FULL)], page_size=4, num_pages=24,
                      max_requests=5)
    live, next_id, reused_before = {}, 0, 0
    for _ in range(600):
        op = rng.random()
        if op < 0.25 and cm.num_free_slots:
            live[next_id] = cm.admit(next_id)
            next_id += 1
        elif op < 0.8 and live:
            rc = live[rng.choice(list(live))]
            n = rng.randint(1, 9)
            if cm.can_extend(rc, n):
                cm.extend(rc, n)
                if rng.random() < 0.9:
                    cm.commit(rc, n)
                else:
                    cm.cancel_reservation(rc)
            else:
                with pytest.raises(OutOfPagesError):
                    cm.extend(rc, n)
        elif live:
            rid = rng.choice(list(live))
            cm.release(live.pop(rid))
        cm.check_invariants()
        for g in cm.groups:
            assert g.pool.num_free + g.pool.num_used == 24
    for rc in live.values():
        cm.release(rc)
    cm.check_invariants()
    assert cm.free_pages() == [24, 24] and cm.num_free_slots == 5
    assert all(g.pool.reuses > 0 for g in cm.groups)


def test_pools_sized_group_by_group():
    """A group with a window gives pages back as the window passes them, so it
    gets by with a pool of a few pages beside a group that keeps every key."""
    needs = [need(0, FULL), need(1, WIN), need(2, FULL)]
    cm = CacheManager(needs, page_size=4, num_pages=[40, 6], max_requests=2)
    assert cm.group_pages == [40, 6] and cm.free_pages() == [40, 6] and cm.pad_pages() == [40, 6]
    assert cm.layer_caches[0].num_pages == 41 and cm.layer_caches[1].num_pages == 7
    # 150 tokens fed 8 at a time: the full group needs 38 pages, the windowed one at most
    # pages_for(10 + 8) + 1 = 6 at any time
    assert cm.peak_pages(150, 8) == [38, 6] and cm.could_ever_hold(150, 8)
    assert not cm.could_ever_hold(150, 16) and not cm.could_ever_hold(170, 8)
    rc = cm.admit("a")
    fed = 0
    while fed < 150:
        n = min(8, 150 - fed)
        cm.extend(rc, n)
        assert cm.free_pages()[1] >= 0
        cm.commit(rc, n)
        fed += n
        cm.check_invariants()
    assert cm.free_pages()[0] == 40 - 38 and cm.free_pages()[1] >= 2
    cm.release(rc)
    assert cm.free_pages() == [40, 6]
    # a function of the group's needs works too; a list of the wrong length is refused
    by_need = CacheManager(needs, page_size=4, num_pages=lambda spec: 5 if spec.window else 30, max_requests=1)
    assert by_need.group_pages == [30, 5]
    with pytest.raises(CacheError, match="cache groups"):
        CacheManager(needs, page_size=4, num_pages=[40, 6, 3], max_requests=2)
    with pytest.raises(CacheError, match="cache groups"):
        CacheManager(needs, page_size=4, num_pages=[40], max_requests=2)


def test_pools_sized_from_free_memory_need_a_device():
    from infernum_b200.errors import CacheError
    need = SimpleNamespace(position=0, paged=PagedCacheSpec(1, 8, 0), state=None, cache_of=None)
    with pytest.raises(CacheError, match="free memory"):
        CacheManager([need], page_size=4, num_pages=None, max_requests=2)
