"""The step function: one batch of (request, its next tokens) in, float32 logits at the
wanted places out.

A batch may hold portions of prompts beside single decoded tokens, cut anywhere.  Only the
tokens given are run; everything earlier comes from the cache, through the block tables that
the cache manager keeps.  Reference: `Engine::run` / `forward_logits`
(crates/engine/src/lib.rs:95-181) with the batch checks of `CudaBackend::metadata`
(crates/kernels/src/lib.rs:407-474); unlike the reference, logits are produced for any wanted
position, not only the last row of a sequence."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Sequence

import numpy as np
import torch

from ..cache.manager import CacheGroup, CacheManager
from ..cache.storage import CacheStorage, bytes_per_page, plan_groups
from ..config.runtime_config import RuntimeConfig
from ..errors import BackendError, InvalidRequest
from ..models.model import Model
from ..models.registry import load_config, model_spec_for
from ..parts.base import Runtime
from ..weights.loader import load_weights
from ..weights.random_init import random_weights
from .context import StepContext


@dataclass
class SequenceStep:
    """The next tokens of one request.  `want` are places among these tokens (0-based) whose
    logits the caller asks for; it may be empty."""

    request_id: int
    tokens: Sequence[int]
    start_pos: int
    want: Sequence[int] = field(default_factory=tuple)


def _align(n: int) -> int:
    return (n + 3) & ~3


def resolve_dtype(dtype) -> torch.dtype:
    names = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
             torch.bfloat16: torch.bfloat16, torch.float32: torch.float32}
    if dtype not in names:
        raise InvalidRequest(f"dtype must be bfloat16 or float32, got {dtype!r}")
    return names[dtype]


class ModelRunner:
    """Owns the model, the device memory of the cache and the cache manager, and runs steps."""

    def __init__(self, config, tensors: dict[str, torch.Tensor], runtime: Runtime, limits: RuntimeConfig,
                 kv_bytes: int | None = None, num_pages: int | None = None, spec=None):
        if not torch.cuda.is_available() or runtime.device.type != "cuda":
            raise BackendError("the engine runs on a CUDA device only; none is available")
        limits.validate()
        if limits.max_seq_len > config.max_position_embeddings:
            raise InvalidRequest("invalid configured context length/page size: max_seq_len "
                                 f"{limits.max_seq_len} exceeds max_position_embeddings "
                                 f"{config.max_position_embeddings}")
        self.config, self.runtime, self.limits = config, runtime, limits
        self.device = runtime.device
        self.model = Model(spec or model_spec_for(config), tensors, runtime)
        kv_needs, state_needs = self.model.kv_needs(), self.model.state_needs()
        keys, group_of = plan_groups(kv_needs)
        if not keys:                       # a model without paged caches still has block tables of width 0
            keys = [("full", 0)]
        element = 4 if runtime.dtype is torch.float32 else 2
        groups = []
        for g, (kind, window) in enumerate(keys):
            per_page = bytes_per_page(kv_needs, group_of, g, limits.page_size, element)
            if num_pages is not None:
                pages = int(num_pages)
            elif kind == "window":
                span = window - 1 + limits.prefill_budget
                pages = limits.max_running * (-(-span // limits.page_size) + 1)
            else:
                if kv_bytes is None:
                    raise InvalidRequest("give kv_bytes or num_pages")
                pages = int(kv_bytes) // max(per_page, 1)
            if pages <= 0 or pages > 2**31 - 1:
                raise InvalidRequest("invalid KV memory budget")
            groups.append(CacheGroup(kind, window, pages))
        self.groups = groups
        self.cache = CacheManager(groups, limits.page_size, limits.max_running)
        self.storage = CacheStorage(kv_needs, state_needs, groups, group_of, limits.max_running, runtime)
        self._host = None       # pinned int32 staging buffer
        self._dev = None
        self.steps = 0
        self.h2d_bytes = 0      # bytes of batch metadata copied to the device so far

    # ------------------------------------------------------------------ construction
    @classmethod
    def load(cls, folder: str, dtype="bfloat16", device="cuda:0", limits: RuntimeConfig | None = None,
             kv_bytes: int | None = None, num_pages: int | None = None) -> "ModelRunner":
        config = load_config(folder)
        spec = model_spec_for(config)
        runtime = Runtime(torch.device(device), resolve_dtype(dtype), (limits or RuntimeConfig()).page_size)
        tensors = load_weights(folder, spec.weight_specs(), runtime.dtype, runtime.device, spec.ignorable_weights)
        return cls(config, tensors, runtime, limits or RuntimeConfig(), kv_bytes, num_pages, spec)

    @classmethod
    def from_random(cls, config, seed: int, dtype="bfloat16", device="cuda:0", limits: RuntimeConfig | None = None,
                    kv_bytes: int | None = None, num_pages: int | None = None) -> "ModelRunner":
        """A model with seeded random weights drawn on the device (no files)."""
        spec = model_spec_for(config)
        runtime = Runtime(torch.device(device), resolve_dtype(dtype), (limits or RuntimeConfig()).page_size)
        tensors = random_weights(spec.weight_specs(), seed, runtime.dtype, runtime.device)
        return cls(config, tensors, runtime, limits or RuntimeConfig(), kv_bytes, num_pages, spec)

    # ------------------------------------------------------------------ one step
    def _staging(self, n: int):
        if self._host is None or self._host.numel() < n:
            size = max(4096, 1 << (n - 1).bit_length())
            self._host = torch.empty(size, dtype=torch.int32, pin_memory=True)
            self._dev = torch.empty(size, dtype=torch.int32, device=self.device)
        return self._host, self._dev

    def build_context(self, sequences: Sequence[SequenceStep]) -> StepContext:
        if not sequences:
            raise InvalidRequest("empty batch or KV pool")
        S, vocab = self.limits.page_size, self.config.vocab_size
        seen = set()
        counts, tables = [], [[] for _ in self.groups]
        for s in sequences:
            n = len(s.tokens)
            if n == 0 or s.start_pos < 0 or s.start_pos + n > self.limits.max_seq_len:
                raise InvalidRequest("batch sequence length/page coverage mismatch")
            if s.request_id in seen:
                raise InvalidRequest("aliased KV write slots in batch: a request appears twice")
            seen.add(s.request_id)
            for wpos in s.want:
                if not 0 <= wpos < n:
                    raise InvalidRequest(f"wanted place {wpos} outside the {n} tokens of the step")
            counts.append(n)
            need_pages = -(-(s.start_pos + n) // S)
            for g in range(len(self.groups)):
                table = self.cache.table(s.request_id, g)
                if table.size < need_pages:
                    raise InvalidRequest("batch sequence length/page coverage mismatch")
                if (table[s.start_pos // S:need_pages] < 0).any():
                    raise InvalidRequest("a page to be written was given back already")
                tables[g].append(table)
        T, B = int(sum(counts)), len(sequences)
        R = sum(len(s.want) for s in sequences)
        widths = [max(max(t.size for t in tables[g]), 1) for g in range(len(self.groups))]
        layout, cursor = {}, 0

        def take(name, n):
            nonlocal cursor
            layout[name] = (cursor, n)
            cursor += _align(n)

        for name, n in (("ids", T), ("pos", T), ("seq", T), ("q_start", B + 1), ("ctx_len", B), ("slot", B), ("want", R)):
            take(name, n)
        for g in range(len(self.groups)):
            take(f"table{g}", B * widths[g])
            take(f"slots{g}", T)
        host, dev = self._staging(cursor)
        buf = host.numpy()

        def view(name):
            start, n = layout[name]
            return buf[start:start + n]

        ids, pos, seq = view("ids"), view("pos"), view("seq")
        q_start, ctx_len, slot, want = view("q_start"), view("ctx_len"), view("slot"), view("want")
        row, w = 0, 0
        host_q_start, host_start, host_slots, fresh = [0], [], [], []
        for i, s in enumerate(sequences):
            n = counts[i]
            tokens = np.asarray(s.tokens, dtype=np.int64)
            if tokens.min() < 0 or tokens.max() >= vocab:
                raise InvalidRequest("token or page ID out of range")
            ids[row:row + n] = tokens
            pos[row:row + n] = np.arange(s.start_pos, s.start_pos + n)
            seq[row:row + n] = i
            for wpos in s.want:
                want[w] = row + wpos
                w += 1
            ctx_len[i] = s.start_pos + n
            slot[i] = self.cache.slot(s.request_id)
            host_start.append(s.start_pos)
            host_slots.append(int(slot[i]))
            fresh.append(s.start_pos == 0)
            row += n
            q_start[i + 1] = row
            host_q_start.append(row)
        q_start[0] = 0
        for g in range(len(self.groups)):
            table_view = view(f"table{g}").reshape(B, widths[g])
            table_view[:] = -1
            slots_view = view(f"slots{g}")
            row = 0
            for i, s in enumerate(sequences):
                t = tables[g][i]
                table_view[i, :t.size] = t
                p = np.arange(s.start_pos, s.start_pos + counts[i])
                slots_view[row:row + counts[i]] = t[p // S].astype(np.int64) * S + p % S
                row += counts[i]
        dev[:cursor].copy_(host[:cursor], non_blocking=True)
        self.h2d_bytes += 4 * cursor

        def dview(name, shape=None):
            start, n = layout[name]
            t = dev[start:start + n]
            return t.view(shape) if shape else t

        return StepContext(
            num_tokens=T, num_sequences=B, token_ids=dview("ids"), positions=dview("pos"), seq_of_token=dview("seq"),
            q_start=dview("q_start"), context_len=dview("ctx_len"), state_slots=dview("slot"),
            want_rows=dview("want") if R else None,
            block_tables=[dview(f"table{g}", (B, widths[g])) for g in range(len(self.groups))],
            slots=[dview(f"slots{g}") for g in range(len(self.groups))],
            host_q_start=host_q_start, host_start_pos=host_start, host_state_slots=host_slots,
            max_query_len=max(counts), max_context_len=max(s.start_pos + c for s, c in zip(sequences, counts)),
            fresh=fresh)

    def forward(self, sequences: Sequence[SequenceStep]) -> torch.Tensor | None:
        """Runs the batch; returns the logits [wanted, vocab] (float32, on the device) in the
        order of the sequences and of their `want`, or None when nothing is wanted.  The
        kernels are queued, not awaited."""
        ctx = self.build_context(sequences)
        self.steps += 1
        with torch.no_grad():
            return self.model.forward(ctx, self.storage)

    def step(self, sequences: Sequence[SequenceStep]) -> torch.Tensor | None:
        """`forward`, then wait for the device: when it returns, the cache holds the step's
        tokens and pages may be given back (reference: crates/core/src/lib.rs:136-137)."""
        try:
            logits = self.forward(sequences)
            torch.cuda.current_stream().synchronize()
            return logits
        except RuntimeError as e:          # a CUDA failure surfaces as torch's RuntimeError
            raise BackendError(f"step failed on the device: {e}") from e
