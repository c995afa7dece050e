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

from .. import kernels
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


class _Staging:
    """A pinned host buffer and its device twin for a step's int32 facts.  The host side is
    rewritten only after the last copy out of it has finished."""

    def __init__(self, device: torch.device, fixed: bool = False):
        self.device, self.fixed = device, fixed
        self.host = self.dev = self.copied = None

    def reserve(self, n: int):
        if self.host is None or (self.host.numel() < n and not self.fixed):
            size = max(4096, 1 << (n - 1).bit_length())
            self.host = torch.empty(size, dtype=torch.int32, pin_memory=True)
            self.dev = torch.empty(size, dtype=torch.int32, device=self.device)
            self.copied = torch.cuda.Event()
        elif self.host.numel() < n:
            raise BackendError("a recorded step outgrew its context buffers")
        else:
            self.copied.synchronize()
        return self.host, self.dev

    def upload(self, n: int) -> None:
        self.dev[:n].copy_(self.host[:n], non_blocking=True)
        self.copied.record()


class _Recorded:
    """One recorded decode step: its context buffers (fixed addresses), graph and logits."""

    def __init__(self, device: torch.device):
        self.staging = _Staging(device, fixed=True)
        self.ctx = self.graph = self.logits = None
        self.launches = 0          # the engine's own kernels in the recording


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
        self._staging = _Staging(self.device)
        # steps of single decoded tokens are recorded and replayed when every mixer allows it
        self.record_decode = all(getattr(b.mixer, "replayable", False) for b in self.model.blocks)
        self._largest_bucket = min(256, 1 << (limits.max_running - 1).bit_length())
        self._records: dict[tuple[int, int], _Recorded] = {}
        self._graph_pool = None
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
    def _check_batch(self, sequences: Sequence[SequenceStep]):
        """The reference's batch checks (crates/kernels/src/lib.rs:407-474); returns the token
        counts and, per group, the requests' block tables."""
        if not sequences:
            raise InvalidRequest("empty batch or KV pool")
        S = self.limits.page_size
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
        return counts, tables

    def build_context(self, sequences: Sequence[SequenceStep], pad_to: int | None = None,
                      table_widths: list[int] | None = None, staging: _Staging | None = None) -> StepContext:
        """Checks the batch and copies what the kernels need to know about it to the device in
        one transfer.  With `pad_to` (single decoded tokens only) the batch is filled up to that
        many sequences with rows that write nothing and whose results nobody reads, block tables
        get the given fixed widths and every row's logits are produced: the shapes and addresses
        of such a context depend on `pad_to` alone, so its kernels can be recorded once and
        replayed."""
        counts, tables = self._check_batch(sequences)
        S, vocab = self.limits.page_size, self.config.vocab_size
        real = len(sequences)
        B = real if pad_to is None else int(pad_to)
        pads = B - real
        T = int(sum(counts)) + pads
        decode = all(c == 1 for c in counts)
        if pads and not decode:
            raise InvalidRequest("only batches of single decoded tokens can be padded")
        R = B if pad_to is not None else sum(len(s.want) for s in sequences)
        widths = table_widths or [max(max(t.size for t in tables[g]), 1) for g in range(len(self.groups))]
        layout, cursor = {}, 0

        def take(name, n):
            nonlocal cursor
            layout[name] = (cursor, n)
            cursor += _align(n)

        for name, n in (("ids", T), ("pos", T), ("seq", T), ("q_start", B + 1), ("ctx_len", B), ("slot", B), ("want", R),
                        ("tiles", 4 * B if decode else 0)):
            take(name, n)
        for g in range(len(self.groups)):
            take(f"table{g}", B * widths[g])
            take(f"slots{g}", T)
        staging = staging or self._staging
        host, dev = staging.reserve(cursor)
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
            if pad_to is None:
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
        if pads:                               # rows that write nothing: token 0 at position 0, state slot -1
            ids[real:], pos[real:], seq[real:] = 0, 0, np.arange(real, B)
            ctx_len[real:], slot[real:] = 1, -1
            q_start[real + 1:] = np.arange(real + 1, B + 1)
            host_q_start += list(range(real + 1, B + 1))
            host_start += [0] * pads
            host_slots += [-1] * pads
            fresh += [True] * pads
        if pad_to is not None:
            want[:] = np.arange(B)
        if decode:                             # one attention tile per sequence; none for a padding row
            tiles = view("tiles").reshape(B, 4)
            tiles[:] = 0
            tiles[:real, 0] = np.arange(real)
            tiles[:real, 1] = np.arange(real)
            tiles[:real, 2] = 1
        for g in range(len(self.groups)):
            table_view = view(f"table{g}").reshape(B, widths[g])
            table_view[:real] = -1
            table_view[real:] = 0              # a padding row reads page 0 and its result is dropped
            slots_view = view(f"slots{g}")
            slots_view[T - pads:] = -1
            row = 0
            for i, s in enumerate(sequences):
                t = tables[g][i]
                if t.size > widths[g]:
                    raise InvalidRequest("batch sequence length/page coverage mismatch")
                table_view[i, :t.size] = t
                p = np.arange(s.start_pos, s.start_pos + counts[i])
                slots_view[row:row + counts[i]] = t[p // S].astype(np.int64) * S + p % S
                row += counts[i]
        staging.upload(cursor)
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
            fresh=fresh, decode_tiles=dview("tiles", (B, 4)) if decode else None, real_sequences=real)

    def forward(self, sequences: Sequence[SequenceStep]) -> torch.Tensor | None:
        """Runs the batch; returns the logits [wanted, vocab] (float32, on the device) in the
        order of the sequences and of their `want`, or None when nothing is wanted.  The
        kernels are queued, not awaited.  The result is valid until the next call."""
        self.steps += 1
        if self._replayable(sequences):
            return self._forward_recorded(sequences)
        ctx = self.build_context(sequences)
        with torch.no_grad():
            return self.model.forward(ctx, self.storage)

    # ------------------------------------------------------------------ recorded decode steps
    # A step of single decoded tokens launches a few hundred small kernels; queueing them one by
    # one costs more host time than the device needs to run them.  Such a step is therefore
    # recorded once as a CUDA graph per (padded batch size, class of context length) and replayed:
    # the batch is padded to the next power of two with rows that write nothing, every tensor of
    # the recorded context lives at a fixed address, and a step only rewrites their contents.
    def _replayable(self, sequences) -> bool:
        return (self.record_decode and 0 < len(sequences) <= self._largest_bucket
                and all(len(s.tokens) == 1 and len(s.want) == 1 for s in sequences))

    def _forward_recorded(self, sequences) -> torch.Tensor:
        real = len(sequences)
        bucket = 1 << (real - 1).bit_length()
        longest = max(s.start_pos + 1 for s in sequences)
        context_class = max(512, 1 << (longest - 1).bit_length())
        key = (bucket, context_class)
        record = self._records.get(key)
        if record is None:
            record = self._records[key] = _Recorded(self.device)
        widths = [-(-self.limits.max_seq_len // self.limits.page_size)] * len(self.groups)
        ctx = self.build_context(sequences, pad_to=bucket, table_widths=widths, staging=record.staging)
        if record.graph is None:
            ctx.max_context_len = context_class      # launches are planned for the class, not for this step
            record.ctx = ctx
            stream = torch.cuda.current_stream()
            side = torch.cuda.Stream(device=self.device)
            side.wait_stream(stream)
            with torch.no_grad(), torch.cuda.stream(side):
                self.model.forward(ctx, self.storage)          # first use of every kernel outside the recording
            stream.wait_stream(side)
            graph = torch.cuda.CUDAGraph()
            counted = kernels.launch_count
            with torch.no_grad(), torch.cuda.graph(graph, pool=self._graph_pool):
                record.logits = self.model.forward(ctx, self.storage)
            record.launches = kernels.launch_count - counted     # recorded, not run
            kernels.launch_count = counted
            if self._graph_pool is None:
                self._graph_pool = graph.pool()
            record.graph = graph
        record.graph.replay()
        kernels.launch_count += record.launches
        return record.logits[:real]

    def step(self, sequences: Sequence[SequenceStep]) -> torch.Tensor | None:
        """`forward`, then wait for the device: when it returns, the cache holds the step's
        tokens and pages may be given back (reference: crates/core/src/lib.rs:136-137)."""
        try:
            logits = self.forward(sequences)
            torch.cuda.current_stream().synchronize()
            kernels.check_device_errors()
            return logits
        except RuntimeError as e:          # a CUDA failure surfaces as torch's RuntimeError
            raise BackendError(f"step failed on the device: {e}") from e
