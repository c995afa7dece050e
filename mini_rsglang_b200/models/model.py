"""A model built from a `ModelSpec`: parts with their tensors bound, run in the order the
spec gives."""
from __future__ import annotations

import torch

from ..parts.base import Runtime
from .spec import ModelSpec


def plain_or_none(pending):
    """A branch output that the stream does not hold yet, or None when it does (`Prenormed`) or there is none."""
    from ..parts.base import Prenormed

    return None if isinstance(pending, Prenormed) else pending


class Model:
    def __init__(self, spec: ModelSpec, tensors: dict[str, torch.Tensor], runtime: Runtime):
        self.spec = spec
        self.runtime = runtime
        self.embedding, self.blocks, self.final_norm, self.head = spec.build_parts()
        for part in (self.embedding, *self.blocks, self.final_norm, self.head):
            part.bind(tensors, runtime)
        # cache entry that each run of the order reads; runs that borrow a cache write nothing
        self.cache_entry = [e.cache_of if e.cache_of is not None else i for i, e in enumerate(spec.run_order)]
        self.writes_cache = [e.cache_of is None for e in spec.run_order]
        self._cache_parts = [b.cache_part() for b in self.blocks if b.cache_part() is not None]

    def _need(self, entry, which: str):
        part = self.blocks[entry.layer].cache_part()
        return getattr(part, which)() if part is not None and entry.cache_of is None else None

    def kv_needs(self):
        return [self._need(e, "cache_need") for e in self.spec.run_order]

    def state_needs(self):
        return [self._need(e, "state_need") for e in self.spec.run_order]

    def replayable(self) -> bool:
        """Whether steps of single decoded tokens may be recorded: every part that keeps a cache allows it."""
        return all(getattr(b.cache_part(), "replayable", False) for b in self.blocks if b.cache_part() is not None)

    def step_signature(self, facts) -> tuple:
        """What the mixers say decides a step's launches beyond its shapes: every layer's answer, a run of equal
        answers once with its length."""
        out = []
        for part in self._cache_parts:
            signature = part.step_signature(facts)
            if out and out[-1][0] == signature:
                out[-1][1] += 1
            else:
                out.append([signature, 1])
        return tuple((signature, count) for signature, count in out)

    def weight_bytes(self) -> int:
        seen, total = set(), 0
        for part in (self.embedding, *self.blocks, self.final_norm, self.head):
            for t in _tensors_of(part):
                if t.data_ptr() not in seen:
                    seen.add(t.data_ptr())
                    total += t.numel() * t.element_size()
        return total

    def forward(self, ctx, storage) -> torch.Tensor | None:
        """Runs the step's tokens through every layer; float32 logits [wanted, vocab], or None
        when no logits are wanted (the head is then skipped, as in the reference,
        crates/engine/src/lib.rs:132-135)."""
        ctx.shared.clear()           # a context may be run again (a recorded step): nothing of the run before is kept
        stream = self.embedding.forward(ctx)
        if ctx.observe:
            ctx.observe("embedding", stream)
        pending = None
        order = self.spec.run_order
        for index, entry in enumerate(order):
            block = self.blocks[entry.layer]
            ctx.label = f"layer{index}"
            extra = {}
            if block.links_norms:        # the norm that reads the stream after this block
                extra["next_norm"] = self.blocks[order[index + 1].layer].entry_norm if index + 1 < len(order) else self.final_norm
            pending = block.forward(stream, pending, ctx, storage.entries[self.cache_entry[index]],
                                    self.writes_cache[index], **extra)
        if ctx.observe:              # the reference norms every row before it gathers the wanted ones (qwen3.rs:228-233)
            ctx.observe("final_norm", self.final_norm.add_norm(stream, plain_or_none(pending), write_back=False))
        if ctx.want_rows is None:
            return None
        rows = None if ctx.want_every_row else ctx.want_rows
        hidden = self.final_norm.add_norm(stream, pending, rows=rows, write_back=False)
        return self.head.forward(hidden)


def _tensors_of(part, seen=None):
    out = []
    seen = seen if seen is not None else set()
    if id(part) in seen:
        return out
    seen.add(id(part))
    for value in vars(part).values():
        if isinstance(value, torch.Tensor):
            out.append(value)
        elif hasattr(value, "bind") and hasattr(value, "weight_specs"):
            out += _tensors_of(value, seen)
    return out
