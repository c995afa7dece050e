"""The scheduler one step ahead of the tokens: a step is committed with tokens whose values are not known yet
(`UNKNOWN_TOKEN`), the next step is planned and queued, and `resolve` brings the values afterwards.  The decisions
must be those of the scheduler that waits for every token, one step later where a value decides them."""
import random

import pytest

from mini_rsglang_b200 import BackendError, RuntimeConfig
from mini_rsglang_b200.cache import CacheGroup, CacheManager
from mini_rsglang_b200.engine.scheduler import UNKNOWN_TOKEN, Scheduler


def make(pages=64, page_size=4, budget=8, running=4, eos=(7,), prefix_cache=False):
    limits = RuntimeConfig(max_seq_len=64, page_size=page_size, prefill_budget=budget, max_running=running, max_waiting=16,
                           prefix_cache=prefix_cache)
    cache = CacheManager([CacheGroup("full", 0, pages)], page_size, running, prefix_cache=prefix_cache)
    return Scheduler(cache, limits, list(eos), 100, "mixed"), cache


def lockstep(s, cache, answer):
    """plan, run, commit with the values: the reference behaviour.  Returns {request: (tokens, reason)}."""
    out, tokens = {}, {}
    for _ in range(200):
        plan = s.plan()
        for f in s.drain():
            out[f.request_id] = (tokens.pop(f.request_id, []), f.reason)
        if not plan:
            break
        sampled = []
        for p in plan:
            if p.sample:
                t = answer(p.request_id, p.start_pos + len(p.tokens))
                sampled.append(t)
                tokens.setdefault(p.request_id, []).append(t)
        s.commit(sampled)
        for f in s.drain():
            out[f.request_id] = (tokens.pop(f.request_id, []), f.reason)
        cache.check_integrity()
    return out


def one_ahead(s, cache, answer):
    """plan, queue, resolve the step before, commit as unknown: the values arrive a step late."""
    out, tokens = {}, {}
    in_flight = None                # (requests, values) of the step that is "still running"
    for _ in range(400):
        plan = s.plan()
        for f in s.drain():
            out[f.request_id] = (tokens.pop(f.request_id, []), f.reason)
        if not plan and in_flight is None:
            break
        now = None
        if plan:
            requests, values = [], []
            for p in plan:
                # a decoded token whose value is still unknown is planned as UNKNOWN_TOKEN: the caller takes it from the device
                if len(p.tokens) == 1 and p.tokens[0] == UNKNOWN_TOKEN:
                    assert in_flight is not None and p.request_id in in_flight[0]
                else:
                    assert all(t >= 0 for t in p.tokens)
                if p.sample:
                    requests.append(p.request_id)
                    values.append(answer(p.request_id, p.start_pos + len(p.tokens)))
            now = (requests, values)
        if in_flight is not None:
            s.resolve(*in_flight)
            for r, t in zip(*in_flight):
                tokens.setdefault(r, []).append(t)
            for f in s.drain():
                kept = tokens.pop(f.request_id, [])
                out[f.request_id] = (kept[:f.completion_tokens], f.reason)
        if plan:
            s.commit([UNKNOWN_TOKEN] * len(now[0]))
        in_flight = now
        cache.check_integrity()
    assert s.idle()
    return out


def traffic(seed):
    rng = random.Random(seed)
    return [([rng.randrange(10, 90) for _ in range(rng.randrange(1, 20))], rng.randrange(1, 9), rng.random() < 0.3)
            for _ in range(rng.randrange(3, 9))]


@pytest.mark.parametrize("seed", range(8))
def test_one_step_ahead_ends_every_request_as_lockstep_does(seed):
    """The answers depend on (request, position) alone, with stop tokens among them: both ways of driving the
    scheduler must give every request the same tokens and the same reason."""
    def answer(request, position):
        return 7 if (request * 31 + position * 17 + seed) % 11 == 0 else 10 + (request * 7 + position) % 80

    results = []
    for drive in (lockstep, one_ahead):
        s, cache = make(pages=24, prefix_cache=seed % 2 == 1)
        for i, (prompt, max_tokens, ignore) in enumerate(traffic(seed)):
            s.submit(i + 1, prompt, max_tokens=max_tokens, ignore_eos=ignore)
        results.append(drive(s, cache, answer))
        cache.clear_idle_cache()
        assert cache.free_pages() == 24 and cache.open_requests() == 0
    assert results[0] == results[1]
    assert {reason for _, reason in results[0].values()} <= {"stop", "length"}


def test_a_stop_token_found_late_drops_the_step_that_was_queued_meanwhile():
    s, cache = make()
    s.submit(1, [11, 12, 13], max_tokens=5)
    assert [(p.start_pos, len(p.tokens), p.sample) for p in s.plan()] == [(0, 3, True)]
    s.commit([UNKNOWN_TOKEN])
    plan = s.plan()                                   # one step ahead: the unknown token is decoded
    assert [(p.start_pos, p.tokens, p.sample) for p in plan] == [(3, [UNKNOWN_TOKEN], True)]
    s.resolve([1], [7])                               # ... and turns out to be the stop token
    done = s.drain()
    assert [(f.request_id, f.reason, f.completion_tokens) for f in done] == [(1, "stop", 1)]
    s.commit([UNKNOWN_TOKEN])                         # the queued step's token belongs to nobody
    assert s.idle() and cache.free_pages() == 64 and not s.plan()
    cache.check_integrity()


def test_max_tokens_is_not_planned_past_and_ends_when_the_value_arrives():
    s, cache = make()
    s.submit(1, [11, 12], max_tokens=2, ignore_eos=True)
    s.plan()
    s.commit([UNKNOWN_TOKEN])
    assert len(s.plan()) == 1
    s.resolve([1], [33])
    s.commit([UNKNOWN_TOKEN])                         # the second and last token
    assert s.plan() == [] and not s.idle() and s.drain() == []       # nothing to run, but the request waits for its value
    s.resolve([1], [34])
    done = s.drain()
    assert [(f.reason, f.completion_tokens) for f in done] == [("length", 2)] and s.idle()
    assert s.counters()["generated_tokens"] == 2 and cache.free_pages() == 64


def test_misuse_is_refused():
    s, cache = make()
    s.submit(1, [11, 12], max_tokens=4, ignore_eos=True)
    s.plan()
    s.commit([UNKNOWN_TOKEN])
    s.plan()
    with pytest.raises(BackendError):
        s.commit([UNKNOWN_TOKEN])                     # a second unknown token of the same request
    s2, _ = make()
    s2.submit(1, [11, 12], max_tokens=4)
    s2.plan()
    s2.commit([20])
    with pytest.raises(BackendError):
        s2.resolve([1], [21])                         # nothing of it is unknown
    s2.resolve([99], [21])                            # a request that is gone is passed over


def test_a_cancel_and_a_failure_with_a_token_outstanding():
    s, cache = make()
    s.submit(1, [11, 12, 13], max_tokens=5, ignore_eos=True)
    s.submit(2, [21, 22], max_tokens=5, ignore_eos=True)
    s.plan()
    s.commit([UNKNOWN_TOKEN, UNKNOWN_TOKEN])
    s.cancel(1)
    plan = s.plan()                                   # the cancelled request ends here, its value never looked at
    assert [p.request_id for p in plan] == [2]
    s.resolve([1, 2], [40, 41])
    s.commit([UNKNOWN_TOKEN])
    s.fail("error")
    reasons = {f.request_id: f.reason for f in s.drain()}
    assert reasons == {1: "cancelled", 2: "error"} and cache.free_pages() == 64
    cache.check_integrity()
