"""Chooses the next token of every sampled row on the device.

Greedy rows take the arg-max (the smaller id wins a tie, crates/kernels/src/ops.cu:152-162).
Other rows are drawn from the reference's support (temperature, then top_k, then top_p;
crates/engine/src/lib.rs:207-244) with a counter-based generator: the n-th token of a
request is drawn with u(seed, n), whatever else is in the batch.  Where the reference keeps
a ChaCha8 stream per request, the per-request state here is the draw count alone."""
from __future__ import annotations

from typing import Sequence

import torch

from .. import kernels
from ..errors import BackendError
from .params import SamplingParams

_MASK64 = (1 << 64) - 1


def uniform_from_counter(seed: int, index: int) -> float:
    """The kernel's u in [0, 1) for (seed, draw index), bit for bit (splitmix64 finaliser)."""
    z = (seed + 0x9E3779B97F4A7C15 * (index + 1)) & _MASK64
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK64
    z ^= z >> 31
    return (z >> 40) / 16777216.0


class Chosen:
    """Tokens that `Sampler.launch` chose: on the device (`tokens`, for a step that goes on before the host has
    seen them) and on their way to pinned host memory (`host`, complete when `arrived` has happened)."""

    def __init__(self, tokens: torch.Tensor, host: torch.Tensor, arrived: torch.cuda.Event):
        self.tokens, self.host, self.arrived = tokens, host, arrived


class Sampler:
    def __init__(self, device: torch.device):
        self.device = device
        self._pinned: list[torch.Tensor] = []       # host buffers that take turns: two results may be outstanding
        self._turn = 0

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams], draw_index: Sequence[int]) -> list[int]:
        """One token per row of `logits` [rows, vocab] (float32, on the device)."""
        return self.read(self.launch(logits, params, draw_index))

    def read(self, chosen: Chosen) -> list[int]:
        """Waits for tokens that `launch` chose and returns them."""
        chosen.arrived.synchronize()
        tokens = chosen.host.tolist()
        if any(t < 0 for t in tokens):
            raise BackendError("empty/nonfinite logits")
        return tokens

    def launch(self, logits: torch.Tensor, params: Sequence[SamplingParams], draw_index: Sequence[int]) -> Chosen:
        """Queues the choice of one token per row of `logits` (int32; a row without finite logits gives -1) and
        their copy to the host, right behind it in the stream, so that work queued later does not hold the copy
        up.  Nothing is waited for."""
        rows = logits.shape[0]
        assert rows == len(params) == len(draw_index)
        out = torch.empty(rows, dtype=torch.int32, device=self.device)
        if all(p.is_greedy() for p in params):
            kernels.argmax(logits, out)
        else:
            # seeds are sent as signed 64-bit patterns of the unsigned value
            seeds = torch.tensor([p.seed - (1 << 64) if p.seed >= (1 << 63) else p.seed for p in params],
                                 dtype=torch.int64)
            temperature = torch.tensor([0.0 if p.is_greedy() else float(p.temperature) for p in params],
                                       dtype=torch.float32)
            top_k = torch.tensor([p.top_k or 0 for p in params], dtype=torch.int32)
            top_p = torch.tensor([float(p.top_p) for p in params], dtype=torch.float32)
            draws = torch.tensor(list(draw_index), dtype=torch.int32)
            dev = self.device
            kernels.sample(logits, temperature.to(dev), top_k.to(dev), top_p.to(dev), seeds.to(dev), draws.to(dev), out)
        while len(self._pinned) < 3:
            self._pinned.append(torch.empty(max(256, rows), dtype=torch.int32, pin_memory=True))
        self._turn = (self._turn + 1) % 3
        if self._pinned[self._turn].numel() < rows:
            self._pinned[self._turn] = torch.empty(2 * rows, dtype=torch.int32, pin_memory=True)
        host = self._pinned[self._turn][:rows]
        host.copy_(out, non_blocking=True)
        arrived = torch.cuda.Event()
        arrived.record()
        return Chosen(out, host, arrived)
