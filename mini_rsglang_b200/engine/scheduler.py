"""The continuous-batching scheduler as Python sees it: a ctypes layer over the native one
(`csrc/host/scheduler.{h,cc}`), which holds the queues, the token histories and every
decision.  The caller runs the planned batch and answers with the sampled tokens."""
from __future__ import annotations

import ctypes
from dataclasses import dataclass

import numpy as np

from ..cache.manager import EXCEPTION, INVALID, NO_ROOM, TOO_LARGE, CacheManager, host_api, last_error
from ..config.runtime_config import RuntimeConfig
from ..errors import BackendError, CapacityError, InvalidRequest

FINISH_REASONS = ("stop", "length", "cancelled", "error")
POLICIES = {"mixed": 0, "alternate": 1}
UNKNOWN_TOKEN = -1      # committed in place of a token whose step is still running; `resolve` brings the value


@dataclass
class PlannedSequence:
    request_id: int
    slot: int
    start_pos: int
    tokens: list[int]
    sample: bool


@dataclass
class FinishedRequest:
    request_id: int
    reason: str
    prompt_tokens: int
    completion_tokens: int
    cached_tokens: int = 0       # prompt tokens that were found in shared pages and not computed again


class Scheduler:
    def __init__(self, cache: CacheManager, limits: RuntimeConfig, eos_ids: list[int], vocab_size: int,
                 policy: str = "mixed"):
        limits.validate()
        if policy not in POLICIES:
            raise InvalidRequest(f"policy must be one of {sorted(POLICIES)}")
        self.lib = host_api()
        self.cache = cache            # kept alive: the native scheduler points into it
        self.limits = limits
        eos = (ctypes.c_int32 * max(len(eos_ids), 1))(*eos_ids)
        self.handle = self.lib.mrs_sched_create(cache.handle, limits.max_seq_len, limits.prefill_budget,
                                                limits.max_running, limits.max_waiting, eos, len(eos_ids),
                                                POLICIES[policy], vocab_size)
        if not self.handle:
            raise InvalidRequest(f"scheduler: {last_error(self.lib)}")
        cap = limits.max_running + 1
        self._req = np.empty(cap, dtype=np.int64)
        self._slot = np.empty(cap, dtype=np.int32)
        self._start = np.empty(cap, dtype=np.int64)
        self._count = np.empty(cap, dtype=np.int64)
        self._sample = np.empty(cap, dtype=np.int32)
        self._tokens = np.empty(max(limits.prefill_budget, 1), dtype=np.int32)
        self._done = (np.empty(64, dtype=np.int64), np.empty(64, dtype=np.int32), np.empty(64, dtype=np.int64),
                      np.empty(64, dtype=np.int64), np.empty(64, dtype=np.int64))     # buffers of `drain`, which runs twice a step

    def __del__(self):
        handle, self.handle = getattr(self, "handle", None), None
        if handle:
            self.lib.mrs_sched_destroy(handle)

    def submit(self, request_id: int, tokens, max_tokens: int, ignore_eos: bool = False) -> None:
        """Queues a request, or raises: `InvalidRequest` (empty prompt, id outside the vocabulary,
        prompt + max_tokens beyond max_seq_len), `CapacityError` (can never fit the pool; queue full)."""
        arr = np.ascontiguousarray(np.asarray(list(tokens), dtype=np.int64))
        if arr.size and (arr.min() < -2**31 or arr.max() >= 2**31):
            raise InvalidRequest("prompt must contain valid nonempty token IDs")
        arr = arr.astype(np.int32)
        code = self.lib.mrs_sched_submit(self.handle, request_id, arr.ctypes.data, arr.size, int(max_tokens),
                                         int(bool(ignore_eos)))
        if code == 0:
            return
        message = last_error(self.lib)
        if code in (NO_ROOM, TOO_LARGE):
            raise CapacityError(message)
        if code == INVALID:
            raise InvalidRequest(message)
        raise BackendError(message)

    def cancel(self, request_id: int) -> bool:
        return bool(self.lib.mrs_sched_cancel(self.handle, request_id))

    def idle(self) -> bool:
        return bool(self.lib.mrs_sched_idle(self.handle))

    def waiting(self) -> int:
        return self.lib.mrs_sched_waiting(self.handle)

    def running(self) -> int:
        return self.lib.mrs_sched_running(self.handle)

    def plan(self) -> list[PlannedSequence]:
        n = self.lib.mrs_sched_plan(self.handle, self._req.ctypes.data, self._slot.ctypes.data,
                                    self._start.ctypes.data, self._count.ctypes.data, self._sample.ctypes.data,
                                    self._req.size)
        if n < 0:
            raise BackendError(f"scheduler plan: {last_error(self.lib)}")
        if n == 0:
            return []
        counts = self._count[:n].tolist()
        total = sum(counts)
        if total > self._tokens.size:
            self._tokens = np.empty(2 * total, dtype=np.int32)
        got = self.lib.mrs_sched_plan_tokens(self.handle, self._tokens.ctypes.data, self._tokens.size)
        if got != total:
            raise BackendError("scheduler: planned tokens are not available")
        tokens = self._tokens[:total].tolist()
        requests, slots, starts, samples = (self._req[:n].tolist(), self._slot[:n].tolist(), self._start[:n].tolist(),
                                            self._sample[:n].tolist())
        out, at = [], 0
        for i in range(n):
            out.append(PlannedSequence(requests[i], slots[i], starts[i], tokens[at:at + counts[i]], bool(samples[i])))
            at += counts[i]
        return out

    def commit(self, sampled: list[int]) -> None:
        """One token per sampled sequence of the plan, in its order; `UNKNOWN_TOKEN` for a token whose step is still
        running (its value follows with `resolve`, before the request's next token is committed)."""
        arr = np.asarray(sampled, dtype=np.int32)
        code = self.lib.mrs_sched_commit(self.handle, arr.ctypes.data, arr.size)
        if code == EXCEPTION:
            raise BackendError(last_error(self.lib))

    def resolve(self, requests: list[int], tokens: list[int]) -> None:
        """The values of tokens that were committed as `UNKNOWN_TOKEN`: the requests they end are finished here."""
        ids = np.asarray(requests, dtype=np.int64)
        values = np.asarray(tokens, dtype=np.int32)
        if ids.size != values.size:
            raise InvalidRequest("resolve: as many tokens as requests")
        code = self.lib.mrs_sched_resolve(self.handle, ids.ctypes.data, values.ctypes.data, ids.size)
        if code == EXCEPTION:
            raise BackendError(last_error(self.lib))

    def fail(self, reason: str = "error") -> None:
        self.lib.mrs_sched_fail(self.handle, FINISH_REASONS.index(reason))

    def drain(self) -> list[FinishedRequest]:
        """Requests that ended since the last call, in the order they ended."""
        out = []
        req, reason, prompt, done, cached = self._done
        cap = req.size
        while True:
            n = self.lib.mrs_sched_drain_cached(self.handle, req.ctypes.data, reason.ctypes.data, prompt.ctypes.data,
                                                done.ctypes.data, cached.ctypes.data, cap)
            for i in range(max(n, 0)):
                out.append(FinishedRequest(int(req[i]), FINISH_REASONS[int(reason[i])], int(prompt[i]), int(done[i]),
                                           int(cached[i])))
            if n < cap:
                return out

    def counters(self) -> dict[str, int]:
        values = np.zeros(9, dtype=np.int64)
        self.lib.mrs_sched_counters(self.handle, values.ctypes.data)
        names = ("submitted", "completed", "cancelled", "failed", "prompt_tokens", "generated_tokens",
                 "prefill_batches", "decode_batches", "mixed_batches")
        out = dict(zip(names, (int(v) for v in values)))
        out["cached_tokens"] = int(self.lib.mrs_sched_cached_tokens(self.handle))
        return out
