"""Limits of one running engine, with the reference's names, defaults and checks
(crates/core/src/lib.rs:146-187)."""
from __future__ import annotations

from dataclasses import dataclass

from ..errors import InvalidRequest


@dataclass
class RuntimeConfig:
    max_seq_len: int = 4096      # prompt + generated tokens of one request
    page_size: int = 16          # tokens per cache page; a power of two, at most 256
    prefill_budget: int = 512    # tokens of one step (decoded tokens and prompt portions)
    max_running: int = 32        # requests that hold cache pages at the same time
    max_waiting: int = 256       # requests queued before admission
    prefix_cache: bool = False   # requests share the full pages of equal first tokens (the reference's default is on;
                                 # here the entry point leaves it off unless asked, the command line turns it on)
    record_mixed_steps: bool = True   # steps with prompt portions are recorded with fixed shapes and replayed
    overlap_steps: bool = True        # a step is queued before the tokens of the step before it have reached the host

    def validate(self) -> None:
        limits = (self.max_seq_len, self.page_size, self.prefill_budget, self.max_running,
                  self.max_waiting)
        if any((not isinstance(v, int)) or v <= 0 for v in limits):
            raise InvalidRequest("runtime limits must be positive")
        if self.page_size & (self.page_size - 1) or self.page_size > 256:
            raise InvalidRequest("page_size must be a power of two <= 256")
