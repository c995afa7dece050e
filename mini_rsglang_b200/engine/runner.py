"""The step function: one batch of (request, its next tokens) in, float32 logits at the
wanted places out.

A batch may hold portions of prompts beside single decoded tokens, cut anywhere.  Only the
tokens given are run; everything earlier comes from the cache, through the block tables that
the cache manager keeps.  Reference: `Engine::run` / `forward_logits`
(crates/engine/src/lib.rs:95-181) with the batch checks of `CudaBackend::metadata`
(crates/kernels/src/lib.rs:407-474); unlike the reference, logits are produced for any wanted
position, not only the last row of a sequence."""
from __future__ import annotations

import ctypes
import os
from dataclasses import dataclass, field
from typing import Sequence

import numpy as np
import torch

from .. import kernels
from ..cache.manager import CacheGroup, CacheManager, host_api
from ..cache.storage import CacheStorage, bytes_per_page, plan_groups
from ..config.runtime_config import RuntimeConfig
from ..errors import BackendError, InvalidRequest
from ..models.model import Model
from ..models.registry import load_config, model_spec_for
from ..parts.base import Runtime
from ..parts.linear import configure_library_products
from ..weights.loader import load_weights
from ..weights.random_init import random_weights
from .context import StepContext, StepFacts


@dataclass
class SequenceStep:
    """The next tokens of one request.  `want` are places among these tokens (0-based) whose
    logits the caller asks for; it may be empty."""

    request_id: int
    tokens: Sequence[int]
    start_pos: int
    want: Sequence[int] = field(default_factory=tuple)


def resolve_dtype(dtype) -> torch.dtype:
    names = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
             torch.bfloat16: torch.bfloat16, torch.float32: torch.float32}
    if dtype not in names:
        raise InvalidRequest(f"dtype must be bfloat16 or float32, got {dtype!r}")
    return names[dtype]


def step_layout_bound(rows: int, sequences: int, table_width: int, groups: int) -> int:
    """An upper bound of the int32 words that `mrs_step_build` lays out for a step of `rows` tokens in
    `sequences` sequences with block tables `table_width` wide in each of `groups` page groups: per token
    the id, position, sequence and one write slot a group; per sequence the start row, context length, state
    slot, a wanted row and an attention tile; the tables; every array rounded up to four words."""
    return (3 + groups) * (rows + 4) + 8 * (sequences + 4) + (rows + 4) + groups * (sequences * table_width + 4)


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
    """One recorded step: its context buffers (fixed addresses), graph and logits."""

    def __init__(self, device: torch.device):
        self.staging = _Staging(device, fixed=True)
        self.ctx = self.graph = self.logits = None
        self.launches = 0          # the engine's own kernels in the recording
        self.plan_offset = 0       # a step with fixed shapes: where the mixers' plans lie in the staging buffer


def fixed_rows(rows: int) -> int:
    """Rows of a recorded step that holds `rows` real ones: 16, 32, 64, then multiples of 64."""
    return max(16, 1 << (rows - 1).bit_length()) if rows <= 64 else -(-rows // 64) * 64


class ModelRunner:
    """Owns the model, the device memory of the cache and the cache manager, and runs steps."""

    def __init__(self, config, tensors: dict[str, torch.Tensor], runtime: Runtime, limits: RuntimeConfig,
                 kv_bytes: int | None = None, num_pages: int | None = None, spec=None):
        if not torch.cuda.is_available() or runtime.device.type != "cuda":
            raise BackendError("the engine runs on a CUDA device only; none is available")
        limits.validate()
        configure_library_products()       # process-wide: exact float32 accumulation in the library's products, no TF32
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
        if limits.prefix_cache and (any(g.kind != "full" for g in groups) or any(need is not None for need in state_needs)):
            raise InvalidRequest("prefix sharing needs a model whose layers keep all their keys and no state of their "
                                 "own per request: a window of keys or a recurrent state cannot be shared")
        self.cache = CacheManager(groups, limits.page_size, limits.max_running, prefix_cache=limits.prefix_cache)
        self.storage = CacheStorage(kv_needs, state_needs, groups, group_of, limits.max_running, runtime)
        self._staging = _Staging(self.device)
        lib = host_api()
        self._step_build = lib.mrs_step_build_padded
        self._step_build.restype = ctypes.c_int64
        self._step_build.argtypes = [ctypes.c_void_p, ctypes.c_int] + [ctypes.c_void_p] * 6 + [
            ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int64, ctypes.c_int64, ctypes.c_void_p, ctypes.c_int64,
            ctypes.c_void_p]
        self._step_error = lib.mrs_step_last_error
        self._step_error.restype = ctypes.c_char_p
        # mixers written in Python read the requests' state slots from a host list
        self._needs_host_slots = any(need is not None for need in state_needs)
        # steps of single decoded tokens are recorded and replayed when every mixer allows it
        self.record_decode = self.model.replayable()
        self._largest_bucket = min(256, 1 << (limits.max_running - 1).bit_length())
        self._records: dict[tuple, _Recorded] = {}
        self._graph_pool = None
        # steps with prompt portions: recorded with fixed shapes at their key's first use
        self.record_mixed = self.record_decode and limits.record_mixed_steps
        self.max_records = 96
        # Steps of up to this many rows are recorded (prefill of 2,048 tokens, recorded against queued: 0.6B shape 4.29
        # against 3.78 ms, where the host cannot queue 250 kernels in the time they take; 8B shape 25.98 against 25.33 ms).
        self.mixed_rows_max = int(os.environ.get("MRS_MIXED_ROWS_MAX", "2048"))      # the variable: for measuring other limits
        self.steps = 0
        self.recorded_steps = 0     # steps that were replayed from a recording
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
    def _fill_step(self, sequences: Sequence[SequenceStep], pad_to: int | None, table_width: int | None,
                   staging: "_Staging", pad_rows: int = 0, extra: np.ndarray | None = None, carried=None):
        """Checks the batch, lays its facts out in the staging buffer (the host library does both) and
        starts the copy to the device.  `extra`: int32 words that follow the layout in the same copy (the
        mixers' plans of a step with fixed shapes).  `carried` = (rows, index, sampled): token ids that the
        host does not know yet, because the step that sampled them is still running: after the copy, row
        rows[i] of the step's ids gets sampled[index[i]] on the device (`sampled`: that step's int32 tokens).
        Returns the layout, the device buffer, the first positions, the token counts and the words that the
        layout took."""
        if not sequences:
            raise InvalidRequest("empty batch or KV pool")
        n = len(sequences)
        requests = np.fromiter((s.request_id for s in sequences), dtype=np.int64, count=n)
        starts = np.fromiter((s.start_pos for s in sequences), dtype=np.int64, count=n)
        counts = np.fromiter((len(s.tokens) for s in sequences), dtype=np.int32, count=n)
        want_counts = np.fromiter((len(s.want) for s in sequences), dtype=np.int32, count=n)
        if counts.min() <= 0:
            raise InvalidRequest("batch sequence length/page coverage mismatch")
        flat = [t for s in sequences for t in s.tokens] if counts.max() > 1 else [s.tokens[0] for s in sequences]
        tokens = np.asarray(flat, dtype=np.int64)
        if tokens.min() < 0 or tokens.max() >= self.config.vocab_size:
            raise InvalidRequest("token or page ID out of range")
        tokens = tokens.astype(np.int32)
        want = np.asarray([w for s in sequences for w in s.want], dtype=np.int32)
        G = len(self.groups)
        layout = np.zeros(14 + 3 * G, dtype=np.int64)
        widest = table_width or -(-self.limits.max_seq_len // self.limits.page_size)
        # a padded step has `pad_to` rows and sequences whatever the number of real ones: its need, and with it
        # the size of a recorded step's fixed buffers, depends on `pad_to` alone
        if carried is not None:
            rows, index, sampled = carried
            if len(rows) != len(index) or len(rows) > n:
                raise InvalidRequest("carried tokens: a row and an index each, at most one a sequence")
            words = np.asarray(list(rows) + list(index), dtype=np.int32)
        room = (0 if extra is None else int(extra.size)) + 2 * (pad_to or n)   # a buffer of fixed size has room for carried tokens
        if carried is not None:
            extra = words if extra is None else np.concatenate([extra, words])
        more = 0 if extra is None else int(extra.size)
        guess = step_layout_bound(pad_rows or pad_to or int(counts.sum()), pad_to or n, widest, G)
        for _ in range(2):
            host, dev = staging.reserve(guess + room)
            used = self._step_build(self.cache.handle, n, requests.ctypes.data, starts.ctypes.data, counts.ctypes.data,
                                    tokens.ctypes.data, want_counts.ctypes.data, want.ctypes.data, int(pad_to or 0),
                                    int(pad_rows), int(table_width or 0), self.limits.max_seq_len, self.config.vocab_size,
                                    host.data_ptr(), host.numel() - room, layout.ctypes.data)
            if used != -7:
                break
            guess = int(layout[0])
        if used < 0:
            message = self._step_error().decode("utf-8", "replace")
            raise (BackendError if used == -100 else InvalidRequest)(message)
        used = int(used)
        if more:
            host[used:used + more] = torch.from_numpy(extra)
        staging.upload(used + more)
        self.h2d_bytes += 4 * (used + more)
        if carried is not None and len(rows):
            at, count = used + more - 2 * len(rows), len(rows)
            if max(rows) >= int(layout[0]) or min(rows) < 0:
                raise InvalidRequest("carried tokens: a row outside the step")
            kernels.patch_tokens(dev[int(layout[4]):int(layout[4]) + int(layout[0])], dev[at:at + count],
                                 dev[at + count:at + 2 * count], sampled, self.config.vocab_size)
        return layout, dev, starts, counts, used

    def build_context(self, sequences: Sequence[SequenceStep], pad_to: int | None = None,
                      table_width: int | None = None, staging: _Staging | None = None, pad_rows: int = 0,
                      facts: StepFacts | None = None, carried=None) -> StepContext:
        """Checks the batch and copies what the kernels need to know about it to the device in
        one transfer; the checking and the layout are the host library's (`csrc/host/step_batch.cc`).
        With `pad_to` (single decoded tokens only) the batch is filled up to that many sequences
        with rows that write nothing and whose results nobody reads, block tables get the given
        fixed width and every row's logits are produced: the shapes and addresses of such a
        context depend on `pad_to` alone, so its kernels can be recorded once and replayed.
        With `pad_rows` as well (any batch with at most one wanted place a sequence) the step has `pad_to`
        sequences, `pad_rows` rows and `pad_to` wanted rows, the added ones without effect; what the mixers
        planned from `facts` follows the layout in the same copy and is found in `plan_views`."""
        extra = None
        if facts is not None and facts.plans:
            extra = np.concatenate([plan.words() for plan in facts.plans.values()])
        layout, dev, starts, counts, used = self._fill_step(sequences, pad_to, table_width, staging or self._staging,
                                                            pad_rows, extra, carried)
        n, G = len(sequences), len(self.groups)
        T, B, R, decode = (int(v) for v in layout[:4])
        plan_views = None
        if facts is not None:
            plan_views, at = {}, used
            for key, plan in facts.plans.items():
                words = plan.words().size
                plan_views[key] = dev[at:at + words].view(-1, 4)
                at += words
            if not any(len(s.want) for s in sequences):
                R = 0                        # nothing is wanted: the head is skipped

        def dview(offset, count, shape=None):
            t = dev[int(offset):int(offset) + count]
            return t.view(shape) if shape else t

        real = n
        ends = np.cumsum(counts)
        pads = B - real
        return StepContext(
            num_tokens=T, num_sequences=B, token_ids=dview(layout[4], T), positions=dview(layout[5], T),
            seq_of_token=dview(layout[6], T), q_start=dview(layout[7], B + 1), context_len=dview(layout[8], B),
            state_slots=dview(layout[9], B), want_rows=dview(layout[10], R) if R else None,
            block_tables=[dview(layout[12 + 3 * g], B * int(layout[13 + 3 * g]), (B, int(layout[13 + 3 * g]))) for g in range(G)],
            slots=[dview(layout[14 + 3 * g], T) for g in range(G)],
            host_q_start=[0] + ends.tolist() + list(range(int(ends[-1]) + 1, int(ends[-1]) + pads + 1)),
            host_start_pos=starts.tolist() + [0] * pads,
            host_state_slots=[self.cache.slot(s.request_id) for s in sequences] + [-1] * pads if self._needs_host_slots else [],
            max_query_len=int(layout[13 + 3 * G]), max_context_len=int(layout[12 + 3 * G]),
            fresh=(starts == 0).tolist() + [True] * pads,
            decode_tiles=dview(layout[11], 4 * B, (B, 4)) if decode else None, real_sequences=real,
            want_every_row=bool(decode) and R == T, facts=facts, plan_views=plan_views, layout_words=used)

    def forward(self, sequences: Sequence[SequenceStep], observe=None, carried=None) -> torch.Tensor | None:
        """Runs the batch; returns the logits [wanted, vocab] (float32, on the device) in the
        order of the sequences and of their `want`, or None when nothing is wanted.  The
        kernels are queued, not awaited.  The result is valid until the next call.

        `observe(label, tensor)`: called with the tensors [tokens of the step, width] that the reference's
        observer sees, under its labels (crates/models/src/qwen3.rs:174-229: embedding, layerN-input_norm,
        -q_proj, -q_norm, -q_rope, -k_rope, -v_proj, -attn, -swiglu, -output, final_norm); such a step runs
        every one of those stages as a kernel of its own and is never replayed from a recording."""
        self.steps += 1
        if observe is None and self._replayable(sequences):
            return self._forward_recorded(sequences, carried)
        if observe is None and self.record_decode and self.record_mixed:
            shapes = self._fixed_shapes(sequences)
            if shapes is not None:
                return self._forward_fixed(sequences, *shapes, carried=carried)
        ctx = self.build_context(sequences, carried=carried)
        ctx.observe = observe
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

    def _forward_recorded(self, sequences, carried=None) -> torch.Tensor:
        self.recorded_steps += 1
        real = len(sequences)
        bucket = 1 << (real - 1).bit_length()
        longest = max(s.start_pos + 1 for s in sequences)
        context_class = max(512, 1 << (longest - 1).bit_length())
        key = (bucket, context_class)
        record = self._records.get(key)
        if record is None:
            record = self._records[key] = _Recorded(self.device)
        width = -(-self.limits.max_seq_len // self.limits.page_size)
        if record.graph is not None:          # the recorded context's tensors stay where they are: only their contents change
            self._fill_step(sequences, bucket, width, record.staging, carried=carried)
            record.graph.replay()
            kernels.launch_count += record.launches
            return record.logits[:real]
        ctx = self.build_context(sequences, pad_to=bucket, table_width=width, staging=record.staging, carried=carried)
        ctx.max_context_len = context_class      # launches are planned for the class, not for this step
        self._record(record, ctx)
        record.graph.replay()
        kernels.launch_count += record.launches
        return record.logits[:real]

    def _record(self, record: _Recorded, ctx: StepContext) -> None:
        """Runs the context's step once outside a recording (first use of every kernel, scratch buffers at
        their sizes), then records it."""
        record.ctx = ctx
        stream = torch.cuda.current_stream()
        side = torch.cuda.Stream(device=self.device)
        side.wait_stream(stream)
        with torch.no_grad(), torch.cuda.stream(side):
            self.model.forward(ctx, self.storage)
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

    # ------------------------------------------------------------------ recorded steps with prompt portions
    # A step that holds prompt portions launches as many kernels as a decode step, and for a small model the
    # host needs longer to queue them than the device to run them.  Such a step is recorded too, with fixed
    # shapes: rows padded to `fixed_rows`, sequences to a power of two (the added ones without rows), as many
    # wanted rows as sequences, block tables at their full width.  What else decides the launches (how many
    # attention tiles of which kind) the mixers state as the step's signature, planned on the host from the
    # step's facts; their plans travel with the layout in the step's one copy to the device, to addresses that
    # stay.  A recording costs about two queued steps; at most `max_records` are made.
    def _fixed_shapes(self, sequences):
        n = len(sequences)
        if n > self._largest_bucket:
            return None
        q_start, start_pos, longest, wanted = [0], [], 0, 0
        for s in sequences:
            count = len(s.tokens)
            if count <= 0 or len(s.want) > 1:
                return None
            q_start.append(q_start[-1] + count)
            start_pos.append(s.start_pos)
            longest = max(longest, s.start_pos + count)
            wanted += len(s.want)
        if q_start[-1] > self.mixed_rows_max or longest > self.limits.max_seq_len:
            return None
        rows, bucket = fixed_rows(q_start[-1]), 1 << (n - 1).bit_length()
        context_class = max(512, 1 << (longest - 1).bit_length())
        facts = StepFacts(q_start, start_pos, context_class, padded_sequences=bucket, padded_tokens=rows)
        key = (rows, bucket, context_class, wanted > 0, self.model.step_signature(facts))
        if key not in self._records and len(self._records) >= self.max_records:
            return None
        return key, facts, rows, bucket, context_class

    def _forward_fixed(self, sequences, key, facts, rows, bucket, context_class, carried=None):
        self.recorded_steps += 1
        wanted = sum(len(s.want) for s in sequences)
        record = self._records.get(key)
        if record is None:
            record = self._records[key] = _Recorded(self.device)
        width = -(-self.limits.max_seq_len // self.limits.page_size)
        if record.graph is not None:
            extra = np.concatenate([plan.words() for plan in facts.plans.values()]) if facts.plans else None
            used = self._fill_step(sequences, bucket, width, record.staging, rows, extra, carried)[4]
            if used != record.plan_offset:
                raise BackendError("a recorded step's layout moved")
        else:
            ctx = self.build_context(sequences, pad_to=bucket, table_width=width, staging=record.staging, pad_rows=rows,
                                     facts=facts, carried=carried)
            ctx.max_context_len = context_class
            record.plan_offset = ctx.layout_words
            self._record(record, ctx)
        record.graph.replay()
        kernels.launch_count += record.launches
        return record.logits[:wanted] if wanted else None

    def step(self, sequences: Sequence[SequenceStep], observe=None) -> torch.Tensor | None:
        """`forward`, then wait for the device: when it returns, the cache holds the step's
        tokens and pages may be given back (reference: crates/core/src/lib.rs:136-137)."""
        try:
            logits = self.forward(sequences, observe)
            torch.cuda.current_stream().synchronize()
            kernels.check_device_errors()
            return logits
        except RuntimeError as e:          # a CUDA failure surfaces as torch's RuntimeError
            raise BackendError(f"step failed on the device: {e}") from e
