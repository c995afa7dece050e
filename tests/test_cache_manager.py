"""The cache manager: pages are never lost, held twice or freed twice, under any order of
requests (model: the reference's seeded lifetime test with an integrity check after every
operation, crates/cache/src/lib.rs:412-497)."""
import random

import pytest

from mini_rsglang_b200 import CapacityError, InvalidRequest
from mini_rsglang_b200.cache import CacheGroup, CacheManager


def live_pages(m, request, group=0):
    return [int(p) for p in m.table(request, group) if p >= 0]


def test_pages_are_handed_out_in_order_and_reused_after_close():
    m = CacheManager([CacheGroup("full", 0, 6)], page_size=4, max_slots=2)
    assert m.open(1) == 0
    m.extend(1, 9)
    assert list(m.table(1)) == [0, 1, 2] and m.free_pages() == 3
    assert m.open(2) == 1
    m.extend(2, 4)
    assert list(m.table(2)) == [3]
    m.extend(1, 12)                      # still inside page 2
    assert list(m.table(1)) == [0, 1, 2]
    m.close(1)
    assert m.free_pages() == 5
    m.open(3)
    m.extend(3, 8)
    assert sorted(m.table(3)) == [1, 2] or sorted(m.table(3)) == [0, 1] or len(set(m.table(3)) & {0, 1, 2}) == 2
    m.check_integrity()


def test_refusals_change_nothing():
    m = CacheManager([CacheGroup("full", 0, 4)], page_size=4, max_slots=2)
    m.open(1)
    m.extend(1, 12)
    before = list(m.table(1))
    with pytest.raises(CapacityError):
        m.extend(1, 20)                  # would need 5 pages
    assert list(m.table(1)) == before and m.length(1) == 12
    with pytest.raises(InvalidRequest):
        m.open(1)                        # duplicate
    with pytest.raises(InvalidRequest):
        m.extend(9, 4)                   # unknown
    with pytest.raises(InvalidRequest):
        m.extend(1, 8)                   # shrinking
    m.open(2)
    with pytest.raises(CapacityError):
        m.open(3)                        # no state slot left
    m.close(1)
    with pytest.raises(InvalidRequest):
        m.close(1)                       # closing twice gives nothing back twice
    m.check_integrity()
    assert m.free_pages() == 4 and m.free_slots() == 1


def test_promise_at_admission_prevents_over_commitment():
    m = CacheManager([CacheGroup("full", 0, 10)], page_size=4, max_slots=4)
    assert m.open(1, reserve_tokens=24) >= 0       # 6 pages promised
    assert m.reserved_pages() == 6
    assert m.try_open(2, reserve_tokens=20) == -1  # 5 more do not fit now
    assert m.try_open(2, reserve_tokens=44) == -2  # 11 never fit
    assert m.open(2, reserve_tokens=16) >= 0
    assert m.open(3) >= 0                          # no promise: lives on what nobody was promised
    with pytest.raises(CapacityError):
        m.extend(3, 4)                             # every free page is promised
    m.extend(1, 24)
    m.extend(2, 16)
    assert m.free_pages() == 0 and m.reserved_pages() == 0
    m.check_integrity()
    m.close(2)
    m.extend(3, 16)
    m.check_integrity()


def test_window_group_gives_pages_back_while_the_request_runs():
    m = CacheManager([CacheGroup("full", 0, 32), CacheGroup("window", 6, 4)], page_size=4, max_slots=2)
    assert m.worst_case_pages(1, 100, 1) == 3 and m.worst_case_pages(1, 100, 8) == 5
    assert m.try_open(1, reserve_tokens=100, max_step=8) == -2     # the window pool has 4 pages
    m.open(1, reserve_tokens=100, max_step=1)
    length = 0
    held_most = 0
    for _ in range(100):
        length += 1
        m.extend(1, length)
        held_most = max(held_most, len(live_pages(m, 1, 1)))
        # a query at position length - 1 reads keys (length - 1 - 6, length - 1]
        first_key = max(0, length - 6)
        table = m.table(1, 1)
        assert all(table[p // 4] >= 0 for p in range(first_key, length))
        m.trim(1, length)
        m.check_integrity()
    assert held_most <= 3
    assert len(live_pages(m, 1, 0)) == 25 and len(live_pages(m, 1, 1)) <= 3
    table = m.table(1, 1)
    assert (table[: (length - 6 + 1) // 4] == -1).all()
    m.close(1)
    assert m.free_pages(0) == 32 and m.free_pages(1) == 4
    m.check_integrity()


def test_window_pages_are_reused_by_the_same_request():
    m = CacheManager([CacheGroup("window", 4, 3)], page_size=4, max_slots=1)
    m.open(1, reserve_tokens=400, max_step=1)
    seen = set()
    for length in range(1, 401):
        m.extend(1, length)
        m.trim(1, length)
        seen.update(live_pages(m, 1))
    assert seen == {0, 1}          # four keys touch at most two pages; the freed one is taken again
    m.check_integrity()


@pytest.mark.parametrize("seed", [0, 1, 2, 3])
def test_random_lifetimes_keep_every_invariant(seed):
    rng = random.Random(seed)
    groups = [CacheGroup("full", 0, 40), CacheGroup("window", 10, 24)]
    m = CacheManager(groups, page_size=4, max_slots=5)
    live = {}          # request -> (length, promised total or 0)
    next_id = 1
    for _ in range(2000):
        action = rng.random()
        if action < 0.25 and len(live) < 5:
            reserve = rng.choice([0, 0, rng.randint(1, 60)])
            code = m.try_open(next_id, reserve, 8)
            if code >= 0:
                live[next_id] = (0, reserve)
            else:
                assert code in (-1, -2)
            next_id += 1
        elif action < 0.8 and live:
            request = rng.choice(list(live))
            length, reserve = live[request]
            grow = rng.randint(1, 8)
            target = length + grow
            if reserve and target > reserve:
                target = reserve
            if target > length:
                try:
                    m.extend(request, target)
                    m.trim(request, target)
                    live[request] = (target, reserve)
                except CapacityError:
                    assert not reserve, "a promised request ran out of pages"
        elif live:
            request = rng.choice(list(live))
            m.close(request)
            del live[request]
        m.check_integrity()
        assert m.open_requests() == len(live) and m.free_slots() == 5 - len(live)
        # no page is in two tables
        for g in range(2):
            pages = [p for r in live for p in live_pages(m, r, g)]
            assert len(pages) == len(set(pages))
            assert len(pages) + m.free_pages(g) == groups[g].num_pages
    for request in list(live):
        m.close(request)
    m.check_integrity()
    assert m.free_pages(0) == 40 and m.free_pages(1) == 24 and m.reserved_pages(0) == 0 and m.reserved_pages(1) == 0
