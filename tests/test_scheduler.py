"""The scheduler's decisions against a fake step function that always answers with a fixed
token (model: the reference's scheduler tests with a fake `ModelRunner`,
crates/runtime/src/scheduler.rs:362-636)."""
import pytest

from mini_rsglang_b200 import CapacityError, InvalidRequest, RuntimeConfig
from mini_rsglang_b200.cache import CacheGroup, CacheManager
from mini_rsglang_b200.engine.scheduler import Scheduler


def make(pages=64, page_size=4, budget=4, running=4, waiting=8, eos=(7,), policy="mixed", max_seq_len=64, vocab=100):
    limits = RuntimeConfig(max_seq_len=max_seq_len, page_size=page_size, prefill_budget=budget, max_running=running,
                           max_waiting=waiting)
    cache = CacheManager([CacheGroup("full", 0, pages)], page_size, running)
    return Scheduler(cache, limits, list(eos), vocab, policy), cache


def run(s, cache, answer=42, steps=100):
    """Drives the scheduler with a fake model; returns the shapes of every planned batch."""
    shapes, finished = [], []
    for _ in range(steps):
        plan = s.plan()
        finished += s.drain()
        if not plan:
            break
        shapes.append([(p.request_id, p.start_pos, len(p.tokens), p.sample) for p in plan])
        s.commit([answer(p) if callable(answer) else answer for p in plan if p.sample])
        finished += s.drain()
        cache.check_integrity()
    return shapes, finished


def test_prompt_is_cut_into_portions_and_only_the_last_samples():
    s, cache = make(budget=4)
    s.submit(1, list(range(10, 20)), max_tokens=2)
    shapes, finished = run(s, cache)
    assert shapes == [[(1, 0, 4, False)], [(1, 4, 4, False)], [(1, 8, 2, True)], [(1, 10, 1, True)]]
    assert [(f.request_id, f.reason, f.prompt_tokens, f.completion_tokens) for f in finished] == [(1, "length", 10, 2)]
    assert cache.free_pages() == 64 and s.idle()


def test_decoded_tokens_share_a_step_with_prompt_portions():
    s, cache = make(budget=6)
    s.submit(1, [1, 2, 3], max_tokens=4)
    plan = s.plan()
    assert [(p.request_id, len(p.tokens), p.sample) for p in plan] == [(1, 3, True)]
    s.commit([42])
    s.submit(2, list(range(20, 32)), max_tokens=2)
    plan = s.plan()
    # request 1 decodes one token, request 2 gets the rest of the budget
    assert [(p.request_id, p.start_pos, len(p.tokens), p.sample) for p in plan] == [(1, 3, 1, True), (2, 0, 5, False)]
    assert plan[0].tokens == [42] and plan[1].tokens == [20, 21, 22, 23, 24]
    s.commit([42])
    plan = s.plan()
    assert [(p.request_id, p.start_pos, len(p.tokens), p.sample) for p in plan] == [(1, 4, 1, True), (2, 5, 5, False)]
    s.commit([42])
    shapes, finished = run(s, cache)
    assert shapes[0] == [(1, 5, 1, True), (2, 10, 2, True)]
    assert {f.request_id for f in finished} == {1, 2}
    c = s.counters()
    assert c["mixed_batches"] >= 3 and c["generated_tokens"] == 6 and c["completed"] == 2


def test_budget_is_shared_in_admission_order():
    s, cache = make(budget=8)
    s.submit(1, list(range(5)), max_tokens=1)
    s.submit(2, list(range(5)), max_tokens=1)
    s.submit(3, list(range(5)), max_tokens=1)
    shapes, _ = run(s, cache)
    assert shapes[0] == [(1, 0, 5, True), (2, 0, 3, False)]
    assert shapes[1] == [(2, 3, 2, True), (3, 0, 5, True)]


def test_alternate_policy_reproduces_homogeneous_batches():
    s, cache = make(budget=4, policy="alternate")
    s.submit(1, [1, 2], max_tokens=3)
    plan = s.plan()
    s.commit([42])
    s.submit(2, list(range(10)), max_tokens=1)
    kinds = []
    for _ in range(8):
        plan = s.plan()
        s.drain()
        if not plan:
            break
        kinds.append({"decode" if p.start_pos >= (2 if p.request_id == 1 else 10) else "prefill" for p in plan})
        s.commit([42 for p in plan if p.sample])
    assert all(len(k) == 1 for k in kinds)                      # never both kinds in one batch
    assert kinds[:4] == [{"decode"}, {"prefill"}, {"decode"}, {"prefill"}]


def test_eos_ends_without_another_step_and_ignore_eos_goes_on():
    s, cache = make(eos=(7,))
    s.submit(1, [1, 2, 3], max_tokens=5)
    s.submit(2, [1, 2, 3], max_tokens=3, ignore_eos=True)
    shapes, finished = run(s, cache, answer=7)
    reasons = {f.request_id: (f.reason, f.completion_tokens) for f in finished}
    assert reasons == {1: ("stop", 1), 2: ("length", 3)}
    assert all(r != 1 for step in shapes[1:] for (r, *_rest) in step)


def test_tiny_pool_makes_the_second_request_wait_at_the_head():
    s, cache = make(pages=5, page_size=4, budget=16)
    s.submit(1, list(range(8)), max_tokens=8)      # 4 pages promised
    s.submit(2, list(range(4)), max_tokens=4)      # 2 pages: must wait
    s.submit(3, [1], max_tokens=1)                 # would fit, but waits behind 2
    plan = s.plan()
    assert [p.request_id for p in plan] == [1] and s.waiting() == 2 and s.running() == 1
    s.commit([42])
    shapes, finished = run(s, cache)
    assert [f.request_id for f in finished] == [1, 2, 3] or [f.request_id for f in finished][0] == 1
    first_with_2 = next(i for i, step in enumerate(shapes) if any(r == 2 for r, *_ in step))
    last_with_1 = max(i for i, step in enumerate(shapes) if any(r == 1 for r, *_ in step))
    assert first_with_2 > last_with_1
    assert cache.free_pages() == 5


def test_refusals_at_submission():
    s, cache = make(pages=4, page_size=4, waiting=2, max_seq_len=32, vocab=50)
    with pytest.raises(InvalidRequest, match="nonempty"):
        s.submit(1, [], 4)
    with pytest.raises(InvalidRequest, match="nonempty"):
        s.submit(1, [1, 50], 4)
    with pytest.raises(InvalidRequest, match="positive"):
        s.submit(1, [1], 0)
    with pytest.raises(InvalidRequest, match="context limit"):
        s.submit(1, list(range(30)), 3)
    with pytest.raises(CapacityError, match="KV capacity"):
        s.submit(1, list(range(10)), 8)              # 5 pages never fit a pool of 4
    s.submit(1, [1, 2], 2)
    with pytest.raises(InvalidRequest, match="duplicate"):
        s.submit(1, [1, 2], 2)
    s.submit(2, [1, 2], 2)
    with pytest.raises(CapacityError, match="queue is full"):
        s.submit(3, [1, 2], 2)
    assert s.counters()["submitted"] == 2


def test_cancel_while_waiting_prefilling_and_decoding():
    s, cache = make(budget=6, running=2)
    s.submit(2, [1, 2], 4)
    s.submit(1, list(range(10)), 4)
    s.submit(3, [1, 2], 4)                           # waits: max_running 2
    s.plan()
    s.commit([42])                                   # request 2 sampled its first token, request 1 is mid-prompt
    assert s.cancel(3) and [f.request_id for f in s.drain()] == [3]
    assert s.cancel(1) and s.cancel(2)
    assert not s.cancel(99)
    plan = s.plan()
    finished = s.drain()
    assert plan == [] and {(f.request_id, f.reason) for f in finished} == {(1, "cancelled"), (2, "cancelled")}
    assert cache.free_pages() == 64 and s.idle()
    assert s.counters()["cancelled"] == 3
    cache.check_integrity()


def test_a_failed_step_returns_every_page():
    s, cache = make(pages=16, budget=8)
    for i in range(1, 6):
        s.submit(i, list(range(6)), 4)
    s.plan()
    s.commit([42])
    s.plan()
    assert cache.free_pages() < 16
    s.fail("error")                                  # the model raised in this step
    finished = s.drain()
    assert sorted(f.request_id for f in finished) == [1, 2, 3, 4, 5] and all(f.reason == "error" for f in finished)
    assert cache.free_pages() == 16 and cache.reserved_pages() == 0 and s.idle()
    assert s.counters()["failed"] == 5
    cache.check_integrity()


def test_wrong_number_of_sampled_tokens_is_an_error():
    from mini_rsglang_b200 import BackendError
    s, cache = make()
    s.submit(1, [1, 2], 2)
    s.plan()
    with pytest.raises(BackendError, match="do not match"):
        s.commit([1, 2])


def test_many_requests_through_a_small_pool_finish_and_free_everything():
    s, cache = make(pages=12, page_size=4, budget=7, running=3, waiting=64)
    import random
    rng = random.Random(3)
    want = {}
    for i in range(1, 41):
        n, m = rng.randint(1, 17), rng.randint(1, 9)
        s.submit(i, [rng.randrange(100) for _ in range(n)], m)
        want[i] = (n, m)
    shapes, finished = run(s, cache, steps=10_000)
    assert sorted(f.request_id for f in finished) == list(range(1, 41))
    assert all(f.reason == "length" and (f.prompt_tokens, f.completion_tokens) == want[f.request_id] for f in finished)
    assert all(sum(n for _, _, n, _ in step) <= 7 for step in shapes)
    assert cache.free_pages() == 12 and cache.free_slots() == 3


def test_load_test_percentile_is_the_reference_s():
    """round((n - 1) * p) of the sorted values (crates/server/src/bench.rs:7-15)."""
    from mini_rsglang_b200.engine.load_test import percentile

    assert percentile([], 0.5) == 0.0
    assert percentile([3.0, 1.0, 2.0], 0.5) == 2.0
    assert percentile([4.0, 1.0, 3.0, 2.0], 0.5) == 3.0          # round(1.5) = 2
    assert percentile(list(range(100)), 0.95) == 94
    assert percentile([0.0, 1.0, 2.0, 3.0, 4.0, 5.0], 0.5) == 3.0    # 2.5 rounds away from zero
