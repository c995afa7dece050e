"""The cache manager as Python sees it: a thin ctypes layer over the native one
(`csrc/host/cache_manager.{h,cc}`), which owns all the bookkeeping."""
from __future__ import annotations

import ctypes
from dataclasses import dataclass

import numpy as np

from ..csrc.build import host_library
from ..errors import BackendError, CapacityError, InvalidRequest

OK, NO_ROOM, TOO_LARGE, UNKNOWN, DUPLICATE, NO_SLOT, INVALID, EXCEPTION = 0, -1, -2, -3, -4, -5, -6, -100

_configured = False


def host_api() -> ctypes.CDLL:
    """The host library with its argument types declared."""
    global _configured
    lib = host_library()
    if _configured:
        return lib
    c_i64, c_int, c_vp = ctypes.c_int64, ctypes.c_int, ctypes.c_void_p
    p_i32, p_i64 = ctypes.POINTER(ctypes.c_int32), ctypes.POINTER(ctypes.c_int64)
    table = {
        "mrs_last_error": (ctypes.c_char_p, []),
        "mrs_cache_create": (c_vp, [c_int, ctypes.POINTER(c_int), ctypes.POINTER(c_int), p_i64, c_int, c_int]),
        "mrs_cache_create_sharing": (c_vp, [c_int, ctypes.POINTER(c_int), ctypes.POINTER(c_int), p_i64, c_int, c_int]),
        "mrs_cache_destroy": (None, [c_vp]),
        "mrs_cache_open_prompt": (c_int, [c_vp, c_i64, c_vp, c_i64, c_i64, c_i64, p_i64]),
        "mrs_cache_publish": (c_int, [c_vp, c_i64, c_vp, c_i64]),
        "mrs_cache_clear_idle": (c_i64, [c_vp]),
        "mrs_cache_shares_prefixes": (c_int, [c_vp]),
        "mrs_cache_cached_pages": (c_i64, [c_vp]),
        "mrs_cache_evictable_pages": (c_i64, [c_vp]),
        "mrs_sched_drain_cached": (c_int, [c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_int]),
        "mrs_sched_cached_tokens": (c_i64, [c_vp]),
        "mrs_cache_open": (c_int, [c_vp, c_i64, c_i64, c_i64]),
        "mrs_cache_extend": (c_int, [c_vp, c_i64, c_i64]),
        "mrs_cache_trim": (c_int, [c_vp, c_i64, c_i64]),
        "mrs_cache_close": (c_int, [c_vp, c_i64]),
        "mrs_cache_table": (c_int, [c_vp, c_i64, c_int, c_vp, c_int]),
        "mrs_cache_slot": (c_int, [c_vp, c_i64]),
        "mrs_cache_length": (c_i64, [c_vp, c_i64]),
        "mrs_cache_free_pages": (c_i64, [c_vp, c_int]),
        "mrs_cache_total_pages": (c_i64, [c_vp, c_int]),
        "mrs_cache_reserved_pages": (c_i64, [c_vp, c_int]),
        "mrs_cache_worst_case_pages": (c_i64, [c_vp, c_int, c_i64, c_i64]),
        "mrs_cache_free_slots": (c_int, [c_vp]),
        "mrs_cache_open_requests": (c_int, [c_vp]),
        "mrs_cache_check": (c_int, [c_vp, ctypes.c_char_p, c_int]),
        "mrs_sched_create": (c_vp, [c_vp, c_i64, c_i64, c_int, c_int, p_i32, c_int, c_int, c_i64]),
        "mrs_sched_destroy": (None, [c_vp]),
        "mrs_sched_submit": (c_int, [c_vp, c_i64, c_vp, c_int, c_i64, c_int]),
        "mrs_sched_cancel": (c_int, [c_vp, c_i64]),
        "mrs_sched_idle": (c_int, [c_vp]),
        "mrs_sched_waiting": (c_int, [c_vp]),
        "mrs_sched_running": (c_int, [c_vp]),
        "mrs_sched_plan": (c_int, [c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_int]),
        "mrs_sched_tokens": (c_int, [c_vp, c_i64, c_i64, c_i64, c_vp]),
        "mrs_sched_plan_tokens": (c_i64, [c_vp, c_vp, c_i64]),
        "mrs_sched_commit": (c_int, [c_vp, c_vp, c_int]),
        "mrs_sched_resolve": (c_int, [c_vp, c_vp, c_vp, c_int]),
        "mrs_sched_fail": (c_int, [c_vp, c_int]),
        "mrs_sched_drain": (c_int, [c_vp, c_vp, c_vp, c_vp, c_vp, c_int]),
        "mrs_sched_counters": (None, [c_vp, c_vp]),
    }
    for name, (restype, argtypes) in table.items():
        fn = getattr(lib, name)
        fn.restype = restype
        fn.argtypes = argtypes
    _configured = True
    return lib


def last_error(lib) -> str:
    return lib.mrs_last_error().decode("utf-8", "replace")


@dataclass(frozen=True)
class CacheGroup:
    """Layers with the same need of the cache: every key ("full") or the last `window`."""

    kind: str = "full"
    window: int = 0
    num_pages: int = 0


class CacheManager:
    """Pages, block tables and state slots of the open requests.

    `open` takes a state slot and, with `reserve_tokens`, a promise of the pages a request of
    that length needs at worst; `extend` makes the pages for the next tokens; `trim` gives back
    what a window has passed; `close` gives back everything.  `check` verifies that no page is
    lost, held twice or freed twice.

    With `prefix_cache` requests share the full pages of equal first tokens (`open_prompt`, `publish`;
    the reference's `--prefix-cache`, crates/cache/src/lib.rs:15-240): pages that only the tree of prefixes
    holds are not free but count as room, and are evicted, least recently used first, when a pool runs short."""

    def __init__(self, groups: list[CacheGroup], page_size: int, max_slots: int, prefix_cache: bool = False):
        if not groups:
            raise InvalidRequest("a cache needs at least one group")
        self.lib = host_api()
        self.groups = list(groups)
        self.page_size = int(page_size)
        self.max_slots = int(max_slots)
        n = len(groups)
        kinds = (ctypes.c_int * n)(*[1 if g.kind == "window" else 0 for g in groups])
        windows = (ctypes.c_int * n)(*[int(g.window) for g in groups])
        pages = (ctypes.c_int64 * n)(*[int(g.num_pages) for g in groups])
        if prefix_cache and any(g.kind != "full" for g in groups):
            raise InvalidRequest("prefix sharing needs layers that keep all their keys: a window of keys cannot be shared")
        create = self.lib.mrs_cache_create_sharing if prefix_cache else self.lib.mrs_cache_create
        self.handle = create(n, kinds, windows, pages, self.page_size, self.max_slots)
        self.prefix_cache = bool(prefix_cache)
        if not self.handle:
            raise InvalidRequest(f"cache manager: {last_error(self.lib)}")
        self._scratch = np.empty(max(int(g.num_pages) for g in groups) + 1, dtype=np.int32)

    def __del__(self):
        handle, self.handle = getattr(self, "handle", None), None
        if handle:
            self.lib.mrs_cache_destroy(handle)

    def _raise(self, code: int, what: str):
        if code == NO_ROOM:
            raise CapacityError(f"{what}: no free page (or promise) left")
        if code == TOO_LARGE:
            raise CapacityError(f"{what}: request exceeds total KV pool capacity")
        if code == NO_SLOT:
            raise CapacityError(f"{what}: every state slot is taken")
        if code == UNKNOWN:
            raise InvalidRequest(f"{what}: unknown request")
        if code == DUPLICATE:
            raise InvalidRequest(f"{what}: request id already open")
        if code == EXCEPTION:
            raise BackendError(f"{what}: {last_error(self.lib)}")
        raise InvalidRequest(f"{what}: invalid arguments")

    def try_open(self, request: int, reserve_tokens: int = 0, max_step: int = 1) -> int:
        """The state slot, or a negative code when the request cannot be opened."""
        return self.lib.mrs_cache_open(self.handle, request, reserve_tokens, max_step)

    def open(self, request: int, reserve_tokens: int = 0, max_step: int = 1) -> int:
        slot = self.try_open(request, reserve_tokens, max_step)
        if slot < 0:
            self._raise(slot, f"open request {request}")
        return slot

    def open_prompt(self, request: int, prompt, reserve_tokens: int, max_step: int = 1) -> tuple[int, int]:
        """Opens a request with its prompt: (state slot, prompt tokens found in shared pages).  The request's
        length starts behind the shared tokens; they are not computed again."""
        tokens = np.ascontiguousarray(prompt, dtype=np.int32)
        shared = ctypes.c_int64(0)
        slot = self.lib.mrs_cache_open_prompt(self.handle, request, tokens.ctypes.data, tokens.size, reserve_tokens,
                                              max_step, ctypes.byref(shared))
        if slot < 0:
            self._raise(slot, f"open request {request}")
        return slot, int(shared.value)

    def publish(self, request: int, tokens, computed: int) -> None:
        """The first `computed` tokens of the request are in its pages: their full pages are shared from now on."""
        tokens = np.ascontiguousarray(tokens, dtype=np.int32)
        if computed > tokens.size:
            raise InvalidRequest("publish: more tokens computed than given")
        code = self.lib.mrs_cache_publish(self.handle, request, tokens.ctypes.data, computed)
        if code < 0:
            self._raise(code, f"publish request {request}")

    def clear_idle_cache(self) -> int:
        """Evicts every page that only the tree of prefixes holds; returns how many."""
        n = int(self.lib.mrs_cache_clear_idle(self.handle))
        if n < 0:
            self._raise(n, "clear the idle cache")
        return n

    def cached_pages(self) -> int:
        return int(self.lib.mrs_cache_cached_pages(self.handle))

    def evictable_pages(self) -> int:
        return int(self.lib.mrs_cache_evictable_pages(self.handle))

    def extend(self, request: int, new_length: int) -> None:
        code = self.lib.mrs_cache_extend(self.handle, request, new_length)
        if code < 0:
            self._raise(code, f"extend request {request} to {new_length} tokens")

    def trim(self, request: int, computed: int) -> int:
        code = self.lib.mrs_cache_trim(self.handle, request, computed)
        if code < 0:
            self._raise(code, f"trim request {request}")
        return code

    def close(self, request: int) -> None:
        code = self.lib.mrs_cache_close(self.handle, request)
        if code < 0:
            self._raise(code, f"close request {request}")

    def table(self, request: int, group: int = 0) -> np.ndarray:
        """Logical page -> physical page of a request in a group (-1: given back)."""
        need = -(-max(int(self.lib.mrs_cache_length(self.handle, request)), 0) // self.page_size)
        if need > self._scratch.size:
            self._scratch = np.empty(2 * need, dtype=np.int32)
        n = self.lib.mrs_cache_table(self.handle, request, group, self._scratch.ctypes.data, self._scratch.size)
        if n < 0:
            self._raise(n, f"block table of request {request}")
        return self._scratch[:n].copy()

    def slot(self, request: int) -> int:
        slot = self.lib.mrs_cache_slot(self.handle, request)
        if slot < 0:
            self._raise(slot, f"slot of request {request}")
        return slot

    def length(self, request: int) -> int:
        n = self.lib.mrs_cache_length(self.handle, request)
        if n < 0:
            self._raise(int(n), f"length of request {request}")
        return int(n)

    def is_open(self, request: int) -> bool:
        return self.lib.mrs_cache_slot(self.handle, request) >= 0

    def free_pages(self, group: int = 0) -> int:
        return int(self.lib.mrs_cache_free_pages(self.handle, group))

    def total_pages(self, group: int = 0) -> int:
        return int(self.lib.mrs_cache_total_pages(self.handle, group))

    def reserved_pages(self, group: int = 0) -> int:
        return int(self.lib.mrs_cache_reserved_pages(self.handle, group))

    def worst_case_pages(self, group: int, tokens: int, max_step: int) -> int:
        return int(self.lib.mrs_cache_worst_case_pages(self.handle, group, tokens, max_step))

    def free_slots(self) -> int:
        return self.lib.mrs_cache_free_slots(self.handle)

    def open_requests(self) -> int:
        return self.lib.mrs_cache_open_requests(self.handle)

    def check(self) -> str:
        """Empty when every invariant holds, else what is broken."""
        buf = ctypes.create_string_buffer(4096)
        self.lib.mrs_cache_check(self.handle, buf, len(buf))
        return buf.value.decode()

    def check_integrity(self) -> None:
        report = self.check()
        if report:
            raise AssertionError(f"cache manager integrity: {report}")
