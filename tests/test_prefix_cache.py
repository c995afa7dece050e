"""Prefix sharing in the cache manager and the scheduler (`csrc/host/prefix_tree.{h,cc}`): requests read the full
pages that earlier requests left for the same first tokens.  Model: the reference's tests of its radix cache and of
the scheduler with it (crates/cache/src/lib.rs:412-497, crates/runtime/src/scheduler.rs:478-492): only full pages
are shared and the last prompt token is always computed; pinned pages are never evicted; the least recently used go
first; under random lifetimes no page is lost, held by strangers or freed twice."""
import random

import pytest

from mini_rsglang_b200 import CapacityError, InvalidRequest, RuntimeConfig
from mini_rsglang_b200.cache import CacheGroup, CacheManager
from mini_rsglang_b200.engine.scheduler import Scheduler


def sharing(pages=32, page_size=4, slots=8, groups=1):
    return CacheManager([CacheGroup("full", 0, pages) for _ in range(groups)], page_size, slots, prefix_cache=True)


def computed(m, request, tokens, length=None):
    """Lets the request 'compute' its tokens (pages made) and publish them."""
    length = len(tokens) if length is None else length
    m.extend(request, length)
    m.publish(request, tokens, length)


def test_only_full_pages_are_shared_and_the_last_token_is_computed():
    m = sharing()
    prompt = list(range(12))
    slot, shared = m.open_prompt(1, prompt, reserve_tokens=16)
    assert shared == 0
    computed(m, 1, prompt)
    first = list(m.table(1))
    # the same prompt again: 12 tokens are 3 full pages, but the last token must be computed, so 2 pages are read
    _, shared = m.open_prompt(2, prompt, reserve_tokens=16)
    assert shared == 8 and m.length(2) == 8 and list(m.table(2)) == first[:2]
    # one token more: the third page is full and is shared too
    _, shared = m.open_prompt(3, prompt + [99], reserve_tokens=20)
    assert shared == 12 and list(m.table(3)) == first[:3]
    # a prompt that leaves the prefix inside the second page shares one page
    _, shared = m.open_prompt(4, prompt[:6] + [77] * 6, reserve_tokens=16)
    assert shared == 4 and list(m.table(4)) == first[:1]
    m.check_integrity()
    m.extend(2, 12)
    assert list(m.table(2))[:2] == first[:2] and m.table(2)[2] not in first      # what it computes goes to a page of its own
    for r in (1, 2, 3, 4):
        m.close(r)
    m.check_integrity()
    assert m.cached_pages() == 3 and m.evictable_pages() == 3 and m.free_pages() == 32 - 3
    assert m.clear_idle_cache() == 3 and m.free_pages() == 32
    m.check_integrity()


def test_pinned_pages_stay_and_the_least_recently_used_go_first():
    m = sharing(pages=8, page_size=2, slots=4)
    a, b = [1, 2, 3, 4, 5], [9, 8, 7, 6, 5]
    for r, prompt in ((1, a), (2, b)):
        m.open_prompt(r, prompt, reserve_tokens=6)
        computed(m, r, prompt)
    m.close(1)
    m.close(2)                                   # 2 + 2 pages remain with the tree, 4 are free
    assert m.cached_pages() == 4 and m.free_pages() == 4
    _, shared = m.open_prompt(3, a, reserve_tokens=6)                 # reads a's pages: they are pinned and used now
    assert shared == 4
    # a request of 5 pages: 4 free + b's 2 evictable; a's 2 are pinned and do not count
    m.open_prompt(4, [50 + i for i in range(10)], reserve_tokens=10)
    m.extend(4, 10)
    assert m.cached_pages() == 3                 # one of b's pages went (its leaf), a's are untouched
    m.check_integrity()
    with pytest.raises(CapacityError):
        m.open_prompt(6, [70 + i for i in range(4)], reserve_tokens=4)       # 2 pages: nothing free, b's page is 1
    m.close(4)
    _, shared_b = m.open_prompt(5, b, reserve_tokens=5)
    assert shared_b == 2                         # b's first page survived its leaf
    m.check_integrity()
    for r in (3, 5):
        m.close(r)
    m.clear_idle_cache()
    assert m.free_pages() == 8
    m.check_integrity()


def test_a_promise_counts_pages_that_can_be_evicted_as_room():
    m = sharing(pages=6, page_size=4, slots=4)
    prompt = list(range(16))
    m.open_prompt(1, prompt, reserve_tokens=16)
    computed(m, 1, prompt)
    m.close(1)
    assert m.free_pages() == 2 and m.evictable_pages() == 4
    # 5 pages for strangers' tokens: 2 free + 3 evicted
    m.open_prompt(2, [100 + i for i in range(20)], reserve_tokens=20)
    m.extend(2, 20)
    assert m.cached_pages() == 1 and m.free_pages() == 0
    m.check_integrity()
    with pytest.raises(CapacityError):
        m.open_prompt(3, [5] * 8, reserve_tokens=8)            # 1 evictable page is not 2
    m.close(2)
    m.check_integrity()


def test_two_page_groups_share_together():
    m = sharing(pages=16, page_size=4, slots=4, groups=2)
    prompt = list(range(9))
    m.open_prompt(1, prompt, reserve_tokens=12)
    computed(m, 1, prompt)
    _, shared = m.open_prompt(2, prompt, reserve_tokens=12)
    assert shared == 8
    assert list(m.table(2, 0)) == list(m.table(1, 0))[:2] and list(m.table(2, 1)) == list(m.table(1, 1))[:2]
    m.close(1)
    m.close(2)
    m.check_integrity()
    assert m.clear_idle_cache() == 2 and m.free_pages(0) == 16 and m.free_pages(1) == 16


def test_sharing_is_refused_for_a_window_of_keys_and_plain_calls_still_work():
    with pytest.raises(InvalidRequest):
        CacheManager([CacheGroup("window", 8, 16)], 4, 2, prefix_cache=True)
    m = sharing()
    m.open(1, reserve_tokens=8)                  # a request without a prompt shares nothing and publishes nothing
    m.extend(1, 8)
    m.close(1)
    assert m.cached_pages() == 0 and m.free_pages() == 32
    plain = CacheManager([CacheGroup("full", 0, 8)], 4, 2)
    assert plain.open_prompt(1, [1, 2, 3, 4, 5], reserve_tokens=8) == (0, 0)    # without a tree: open()
    plain.extend(1, 5)
    plain.publish(1, [1, 2, 3, 4, 5], 5)
    plain.close(1)
    assert plain.free_pages() == 8 and plain.cached_pages() == 0


@pytest.mark.parametrize("seed", [1, 2, 3, 4])
def test_random_lifetimes_with_sharing_keep_every_page_accounted_for(seed):
    """Requests with prompts drawn from a few families (common first pages) open, compute in portions, publish,
    decode and close in random order through a pool that is too small for all of them; after every operation the
    books must balance, and a request must find its own first tokens in what it reads."""
    rng = random.Random(seed)
    page = 4
    m = sharing(pages=40, page_size=page, slots=6)
    families = [[rng.randrange(50) for _ in range(24)] for _ in range(3)]
    content = {}                                 # physical page -> tokens that were "written" there
    live = {}
    next_id = 1
    for _ in range(600):
        op = rng.random()
        if op < 0.35 and len(live) < 6:
            family = rng.choice(families)
            prompt = family[:rng.randrange(1, 24)] + [rng.randrange(50, 60) for _ in range(rng.randrange(0, 6))]
            total = len(prompt) + rng.randrange(1, 8)
            try:
                _, shared = m.open_prompt(next_id, prompt, reserve_tokens=total)
            except CapacityError:
                m.check_integrity()
                continue
            assert shared % page == 0 and shared <= len(prompt) - 1
            table = list(m.table(next_id))
            for i in range(shared // page):      # what it reads holds exactly its own first tokens
                assert content[table[i]] == prompt[i * page:(i + 1) * page]
            live[next_id] = {"tokens": list(prompt), "prompt": len(prompt), "done": shared, "total": total, "published": False}
            next_id += 1
        elif op < 0.85 and live:
            r = rng.choice(list(live))
            state = live[r]
            if state["done"] >= state["total"]:
                continue
            if state["done"] < state["prompt"]:
                end = min(state["prompt"], state["done"] + rng.randrange(1, 9))
            else:
                end = state["done"] + 1
                state["tokens"].append(rng.randrange(60, 70))
            m.extend(r, end)
            table = list(m.table(r))
            for position in range(state["done"], end):           # "write" the tokens into the request's pages
                content.setdefault(table[position // page], [None] * page)
                if position % page == 0:
                    content[table[position // page]] = [None] * page
                content[table[position // page]][position % page] = state["tokens"][position]
            state["done"] = end
            if end >= state["prompt"] and not state["published"]:
                m.publish(r, state["tokens"], state["prompt"])
                state["published"] = True
        elif live:
            r = rng.choice(list(live))
            m.close(r)
            del live[r]
        m.check_integrity()
    for r in list(live):
        m.close(r)
    m.check_integrity()
    m.clear_idle_cache()
    assert m.free_pages() == 40 and m.cached_pages() == 0
    m.check_integrity()


def make(pages=64, page_size=4, budget=8, running=4):
    limits = RuntimeConfig(max_seq_len=64, page_size=page_size, prefill_budget=budget, max_running=running,
                           max_waiting=8, prefix_cache=True)
    cache = CacheManager([CacheGroup("full", 0, pages)], page_size, running, prefix_cache=True)
    return Scheduler(cache, limits, [7], 100, "mixed"), cache


def drive(s, cache):
    shapes, finished = [], []
    for _ in range(100):
        plan = s.plan()
        finished += s.drain()
        if not plan:
            break
        shapes.append([(p.request_id, p.start_pos, len(p.tokens), p.sample) for p in plan])
        s.commit([42 for p in plan if p.sample])
        finished += s.drain()
        cache.check_integrity()
    return shapes, finished


def test_a_repeated_prompt_is_not_computed_again():
    s, cache = make()
    prompt = list(range(10, 23))                 # 13 tokens: 3 full pages
    s.submit(1, prompt, max_tokens=2)
    shapes, finished = drive(s, cache)
    assert shapes[0] == [(1, 0, 8, False)] and finished[0].cached_tokens == 0
    s.submit(2, prompt, max_tokens=2)
    shapes, finished = drive(s, cache)
    # 12 of the 13 prompt tokens lie in shared pages: one token is computed, and it yields the first sample
    assert shapes == [[(2, 12, 1, True)], [(2, 13, 1, True)]]
    assert finished[0].cached_tokens == 12 and finished[0].prompt_tokens == 13
    assert s.counters()["cached_tokens"] == 12
    # a prompt that shares two pages and goes its own way
    s.submit(3, prompt[:9] + [1, 2, 3], max_tokens=1)
    shapes, finished = drive(s, cache)
    assert shapes == [[(3, 8, 4, True)]] and finished[0].cached_tokens == 8
    assert cache.cached_pages() >= 3
    cache.clear_idle_cache()
    assert cache.free_pages() == 64 and s.idle()


def test_a_next_turn_reads_the_prompt_and_the_answer_of_the_turn_before():
    s, cache = make()
    prompt = list(range(10, 20))                 # 10 tokens, pages of 4
    s.submit(1, prompt, max_tokens=7)
    _, finished = drive(s, cache)
    assert finished[0].reason == "length" and finished[0].completion_tokens == 7
    # the request held 10 + 7 tokens, of which the last was sampled and never computed: 16 tokens = 4 full pages stay
    assert cache.cached_pages() == 4
    turn = prompt + [42] * 7 + [50, 51, 52]
    s.submit(2, turn, max_tokens=1)
    shapes, finished = drive(s, cache)
    assert finished[0].cached_tokens == 16 and shapes == [[(2, 16, 4, True)]]
    s.submit(3, prompt, max_tokens=2)
    s.plan()
    s.cancel(3)                                  # a cancelled request publishes nothing beyond its prompt's pages
    s.plan()
    cache.check_integrity()
    cache.clear_idle_cache()
    assert cache.free_pages() == 64


def test_requests_that_run_together_share_what_the_first_has_published():
    s, cache = make(budget=8, running=2)
    prompt = list(range(30, 47))                 # 17 tokens
    s.submit(1, prompt, max_tokens=3)
    s.plan()
    s.commit([])                                 # 8 of 17 tokens: nothing published yet
    s.submit(2, prompt, max_tokens=3)
    shapes, finished = drive(s, cache)
    # request 2 was admitted while request 1's prompt was still open: it found nothing and computes everything
    assert shapes[0][0][:3] == (1, 8, 8) or shapes[0][0][:3] == (1, 8, 8)
    assert {f.request_id: f.cached_tokens for f in finished} == {1: 0, 2: 0}
    s.submit(3, prompt, max_tokens=1)
    shapes, finished = drive(s, cache)
    assert finished[0].cached_tokens == 16 and shapes == [[(3, 16, 1, True)]]
    cache.clear_idle_cache()
    assert cache.free_pages() == 64


def test_a_failed_step_returns_every_page_with_sharing_too():
    s, cache = make()
    prompt = list(range(12))
    s.submit(1, prompt, max_tokens=4)
    drive(s, cache)
    s.submit(2, prompt, max_tokens=4)
    s.submit(3, [5] * 9, max_tokens=4)
    s.plan()
    s.fail("error")
    reasons = {f.request_id: f.reason for f in s.drain()}
    assert reasons == {2: "error", 3: "error"}
    cache.check_integrity()
    cache.clear_idle_cache()
    assert cache.free_pages() == 64 and cache.open_requests() == 0
