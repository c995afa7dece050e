"""Device memory of the cache: for every run of a layer that keeps a cache, key and value
pages `[pages, kv_heads, page_size, head_dim]` in its group's page space, and for every
mixer with a per-request state an array `[slots, *shape]`.  The reference keeps two tensors
`[pages, page_size, kv_heads, head_dim]` per layer (crates/models/src/model.rs:96-120); here
one head's rows of a page are contiguous, so a kernel reads a page of one head as one block."""
from __future__ import annotations

from dataclasses import dataclass

import torch

from ..parts.base import KVNeed, Runtime, StateNeed
from .manager import CacheGroup


@dataclass
class CacheEntry:
    group: int = -1                    # index into the manager's groups (-1: no paged cache)
    k: torch.Tensor | None = None
    v: torch.Tensor | None = None
    state: torch.Tensor | None = None  # [slots, *shape]


def plan_groups(needs: list[KVNeed | None]) -> tuple[list[tuple[str, int]], list[int]]:
    """Distinct (kind, window) among the needs, and each need's group index (-1 for None)."""
    keys: list[tuple[str, int]] = []
    index = []
    for need in needs:
        if need is None:
            index.append(-1)
            continue
        key = (need.kind, need.window if need.kind == "window" else 0)
        if key not in keys:
            keys.append(key)
        index.append(keys.index(key))
    return keys, index


def bytes_per_page(needs: list[KVNeed | None], group_of: list[int], group: int, page_size: int,
                   element_size: int) -> int:
    """Bytes that one page of a group takes over all the layers of the group
    (reference: `kv_bytes_per_page`, crates/models/src/model.rs:28-42)."""
    return sum(2 * n.kv_heads * n.head_dim * page_size * element_size
               for n, g in zip(needs, group_of) if n is not None and g == group)


class CacheStorage:
    def __init__(self, kv_needs: list[KVNeed | None], state_needs: list[StateNeed | None],
                 groups: list[CacheGroup], group_of: list[int], max_slots: int, runtime: Runtime):
        self.entries: list[CacheEntry] = []
        for need, state, g in zip(kv_needs, state_needs, group_of):
            entry = CacheEntry(group=g)
            if need is not None:
                shape = (groups[g].num_pages, need.kv_heads, runtime.page_size, need.head_dim)
                entry.k = torch.zeros(shape, dtype=runtime.dtype, device=runtime.device)
                entry.v = torch.zeros(shape, dtype=runtime.dtype, device=runtime.device)
            if state is not None:
                entry.state = torch.zeros((max_slots, *state.shape), dtype=state.dtype, device=runtime.device)
            self.entries.append(entry)

    def bytes(self) -> int:
        total = 0
        for e in self.entries:
            for t in (e.k, e.v, e.state):
                if t is not None:
                    total += t.numel() * t.element_size()
        return total
