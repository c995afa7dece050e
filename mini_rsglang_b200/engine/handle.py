"""The Python entry point, in the manner of the reference's `EngineHandle`
(crates/runtime/src/lib.rs:83-324; example crates/runtime/examples/generate.rs):

    engine = EngineHandle.load(model_dir, device=0, kv_bytes=2 << 30, config=RuntimeConfig())
    stream = engine.generate(GenerateRequest(TokenIds([1, 2, 3]), SamplingParams(max_tokens=8)))
    for event in stream:      # Token(...), ..., Finished(...)
        ...
    engine.shutdown()

The reference runs its scheduler on a thread of its own and streams events through channels;
here the caller's thread drives the engine: iterating a stream runs scheduler steps until the
stream's next event exists.  Requests submitted before iterating run together (continuous
batching).  Prompts are token ids; there is no tokenizer."""
from __future__ import annotations

import weakref
from collections import deque
from dataclasses import dataclass, field
from typing import Iterator, Sequence

import torch

from .. import kernels
from ..config.runtime_config import RuntimeConfig
from ..errors import BackendError, EngineError, EngineStopped
from ..models.registry import load_config
from ..sampling import Sampler, SamplingParams
from .runner import ModelRunner, SequenceStep
from .scheduler import UNKNOWN_TOKEN, Scheduler


@dataclass
class TokenIds:
    """A prompt given as token ids (`Prompt::TokenIds`, crates/core/src/lib.rs:67-71)."""

    ids: Sequence[int]


@dataclass
class GenerateRequest:
    prompt: TokenIds | Sequence[int]
    sampling: SamplingParams = field(default_factory=SamplingParams)


@dataclass
class Token:
    request_id: int
    token_id: int


@dataclass
class Finished:
    request_id: int
    reason: str               # "stop" | "length" | "cancelled" | "error"
    prompt_tokens: int
    completion_tokens: int
    cached_tokens: int = 0


@dataclass
class Error:
    request_id: int
    message: str


@dataclass
class GenerationResult:
    request_id: int
    token_ids: list[int]
    finish_reason: str
    prompt_tokens: int
    completion_tokens: int
    cached_tokens: int = 0      # prompt tokens read from pages that an earlier request left (prefix sharing)


class GenerationStream:
    """Events of one request.  `cancel()`, leaving a `with` block or dropping the last reference stops the
    request at the next step, as dropping the reference's stream does (crates/runtime/src/lib.rs:78-82)."""

    def __init__(self, engine: "EngineHandle", request_id: int):
        self.engine, self.request_id = engine, request_id
        self.events: deque = deque()
        self.terminal = False

    def cancel(self) -> None:
        if not self.terminal and self.engine.healthy:
            self.engine.scheduler.cancel(self.request_id)

    def __enter__(self) -> "GenerationStream":
        return self

    def __exit__(self, *exc) -> None:
        self.cancel()

    def __del__(self):
        try:
            self.cancel()
        except Exception:       # the interpreter may be shutting down: the scheduler is gone with it
            pass

    def __iter__(self) -> Iterator:
        return self

    def __next__(self):
        while not self.events:
            if self.terminal:
                raise StopIteration
            if not self.engine.run_step() and not self.events and not self.terminal:
                self.terminal = True
                raise StopIteration
        event = self.events.popleft()
        if isinstance(event, (Finished, Error)) and not self.events:
            self.terminal = True
        return event


class _InFlight:
    """A step that has been queued and whose sampled tokens the host has not read yet."""

    def __init__(self, ids: list[int], chosen, done):
        self.ids = ids                                  # requests that sample, in the step's order
        self.place = {request_id: k for k, request_id in enumerate(ids)}
        self.chosen = chosen                            # what the sampler launched (`sampling.sampler.Chosen`), or None
        self.done = done                                # recorded behind the step


class EngineHandle:
    def __init__(self, runner: ModelRunner, eos_ids: list[int], policy: str = "mixed", model_id: str = ""):
        self.runner = runner
        self.config = runner.limits
        self.scheduler = Scheduler(runner.cache, runner.limits, eos_ids, runner.config.vocab_size, policy)
        self.sampler = Sampler(runner.device)
        # the engine does not keep a stream alive: a caller who drops one cancels its request
        self.streams: "weakref.WeakValueDictionary[int, GenerationStream]" = weakref.WeakValueDictionary()
        self.params: dict[int, SamplingParams] = {}
        self.generated: dict[int, int] = {}
        self.next_id = 1
        self.healthy = True
        self._in_flight: _InFlight | None = None
        self.info = {"model_id": model_id, "vocab_size": runner.config.vocab_size,
                     "num_pages": [g.num_pages for g in runner.groups], "dtype": str(runner.runtime.dtype)}

    # ------------------------------------------------------------------ loading
    @classmethod
    def load(cls, model: str, device: int | str = 0, kv_bytes: int = 2048 << 20, config: RuntimeConfig | None = None,
             dtype: str = "bfloat16", num_pages: int | None = None, policy: str = "mixed") -> "EngineHandle":
        import os

        config = config or RuntimeConfig()
        config.validate()
        device = f"cuda:{device}" if isinstance(device, int) else device
        runner = ModelRunner.load(model, dtype=dtype, device=device, limits=config,
                                  kv_bytes=None if num_pages else kv_bytes, num_pages=num_pages)
        eos = load_config(model).eos_ids(model)
        return cls(runner, eos, policy, os.path.basename(os.path.normpath(model)))

    @classmethod
    def from_random(cls, model_config, seed: int, device: int | str = 0, kv_bytes: int = 2048 << 20,
                    config: RuntimeConfig | None = None, dtype: str = "bfloat16", num_pages: int | None = None,
                    policy: str = "mixed") -> "EngineHandle":
        config = config or RuntimeConfig()
        device = f"cuda:{device}" if isinstance(device, int) else device
        runner = ModelRunner.from_random(model_config, seed, dtype=dtype, device=device, limits=config,
                                         kv_bytes=None if num_pages else kv_bytes, num_pages=num_pages)
        return cls(runner, model_config.eos_ids(), policy, f"random-{seed}")

    # ------------------------------------------------------------------ requests
    def generate(self, request: GenerateRequest) -> GenerationStream:
        request.sampling.validate()
        if not self.healthy:
            raise EngineStopped("engine stopped")
        prompt = request.prompt.ids if isinstance(request.prompt, TokenIds) else request.prompt
        request_id = self.next_id
        self.scheduler.submit(request_id, prompt, request.sampling.max_tokens, request.sampling.ignore_eos)
        self.next_id += 1
        stream = GenerationStream(self, request_id)
        self.streams[request_id] = stream
        self.params[request_id] = request.sampling
        self.generated[request_id] = 0
        return stream

    def generate_many(self, prompts: Sequence[Sequence[int]], sampling: SamplingParams | Sequence[SamplingParams]
                      ) -> list[GenerationResult]:
        """Submits every prompt, runs them to the end together, returns results in order."""
        if isinstance(sampling, SamplingParams):
            sampling = [sampling] * len(prompts)
        streams, waiting = [], list(zip(prompts, sampling))
        results: dict[int, GenerationResult] = {}
        tokens: dict[int, list[int]] = {}
        order = []

        def collect():
            for stream in streams:
                while stream.events:
                    event = stream.events.popleft()
                    if isinstance(event, Token):
                        tokens[event.request_id].append(event.token_id)
                    elif isinstance(event, Finished):
                        stream.terminal = True
                        results[event.request_id] = GenerationResult(
                            event.request_id, tokens[event.request_id], event.reason, event.prompt_tokens,
                            event.completion_tokens, event.cached_tokens)
                    elif isinstance(event, Error):
                        raise BackendError(event.message)

        while waiting or len(results) < len(order):
            while waiting and self.scheduler.waiting() < self.config.max_waiting:
                prompt, params = waiting.pop(0)
                stream = self.generate(GenerateRequest(TokenIds(prompt), params))
                streams.append(stream)
                order.append(stream.request_id)
                tokens[stream.request_id] = []
            progressed = self.run_step()
            collect()
            if not progressed and not waiting and len(results) < len(order):
                raise BackendError("scheduler is idle but requests are unfinished")
        return [results[i] for i in order]

    # ------------------------------------------------------------------ one scheduler step
    def _emit_finished(self) -> None:
        for done in self.scheduler.drain():
            stream = self.streams.pop(done.request_id, None)
            self.params.pop(done.request_id, None)
            self.generated.pop(done.request_id, None)
            if stream is not None:
                stream.events.append(Finished(done.request_id, done.reason, done.prompt_tokens, done.completion_tokens,
                                              done.cached_tokens))

    def run_step(self) -> bool:
        """Plans, runs and commits one step.  False when there was nothing to run.

        With `overlap_steps` (the default) a step is queued before the tokens of the step before it have reached
        the host: the scheduler is told of tokens whose values are still unknown, the next step takes them from
        the device (`ModelRunner.forward(carried=...)`), and while it runs the host reads the step before,
        streams its tokens and ends what they end.  Tokens and `Finished` events therefore arrive one step late,
        and a request that a stop token ended has one more row computed in vain.  Cache pages given back while a
        step still runs are safe to hand out: whatever uses them next is queued behind that step."""
        if not self.healthy:
            raise EngineStopped("engine stopped")
        plan = self.scheduler.plan()
        self._emit_finished()
        if not plan:
            if self._in_flight is None:
                return False
            self._guarded(self._resolve_in_flight)          # the last step's tokens
            return True
        self._guarded(self._run_plan, plan)
        return True

    def _guarded(self, work, *args):
        try:
            return work(*args)
        except (EngineError, RuntimeError) as e:
            # a failed step ends every request and gives every page back (scheduler.rs:332-359)
            self.healthy = False
            self._in_flight = None
            message = f"{type(e).__name__}: {e}"
            for stream in list(self.streams.values()):
                stream.events.append(Error(stream.request_id, message))
            self.scheduler.fail("error")
            self._emit_finished()
            raise BackendError(message) from e

    def _run_plan(self, plan) -> None:
        overlap = self.config.overlap_steps
        before = self._in_flight
        batch, rows, index, at = [], [], [], 0
        for p in plan:
            tokens = p.tokens
            if len(tokens) == 1 and tokens[0] == UNKNOWN_TOKEN:       # sampled by the step that is still running
                rows.append(at)
                index.append(before.place[p.request_id])
                tokens = [0]
            batch.append(SequenceStep(p.request_id, tokens, p.start_pos, [len(tokens) - 1] if p.sample else []))
            at += len(tokens)
        sampled_ids = [p.request_id for p in plan if p.sample]
        logits = self.runner.forward(batch, carried=(rows, index, before.chosen.tokens) if rows else None)
        chosen = None
        if sampled_ids:
            chosen = self.sampler.launch(logits, [self.params[i] for i in sampled_ids],
                                         [self.generated[i] for i in sampled_ids])
        done = torch.cuda.Event()
        done.record()
        self._in_flight = _InFlight(sampled_ids, chosen, done)
        if before is not None:
            self._resolve(before)               # the host's share of the step before, while this one runs
        if not overlap:
            self._resolve_in_flight(commit=True)
            return
        self.scheduler.commit([UNKNOWN_TOKEN] * len(sampled_ids))
        for request_id in sampled_ids:
            if request_id in self.generated:    # (not ended by the step before, whose tokens have just arrived)
                self.generated[request_id] += 1

    def _resolve_in_flight(self, commit: bool = False) -> None:
        step, self._in_flight = self._in_flight, None
        self._resolve(step, commit)

    def _resolve(self, step: "_InFlight", commit: bool = False) -> None:
        """Waits for a queued step, reads what it sampled, tells the scheduler and the streams."""
        if step.ids:
            tokens = self.sampler.read(step.chosen)
        else:
            tokens = []
            step.done.synchronize()
        kernels.check_device_errors()
        if commit:                              # in lockstep: the plan is still the scheduler's last
            self.scheduler.commit(tokens)
        else:
            self.scheduler.resolve(step.ids, tokens)
        for request_id, token in zip(step.ids, tokens):
            if commit and request_id in self.generated:
                self.generated[request_id] += 1
            stream = self.streams.get(request_id)
            if stream is not None:
                stream.events.append(Token(request_id, token))
        self._emit_finished()

    # ------------------------------------------------------------------ the rest of the reference's surface
    def metrics(self) -> dict:
        """The reference's counters (crates/runtime/src/metrics.rs:4-20) as a dict."""
        out = self.scheduler.counters()
        cache = self.runner.cache
        by_group = [cache.free_pages(g) for g in range(len(self.runner.groups))]
        out.update(waiting=self.scheduler.waiting(), running=self.scheduler.running(),
                   free_pages=sum(by_group), free_pages_by_group=by_group,
                   total_pages=sum(cache.total_pages(g) for g in range(len(self.runner.groups))),
                   cached_pages=cache.cached_pages() * len(self.runner.groups),
                   peak_memory_bytes=torch.cuda.max_memory_allocated(self.runner.device), healthy=self.healthy)
        return out

    def clear_cache(self) -> None:
        """Gives back every page that only the tree of shared prefixes holds (reference: `clear_idle_cache`,
        crates/cache/src/lib.rs:376-380).  Nothing to do without prefix sharing."""
        self.runner.cache.clear_idle_cache()

    def shutdown(self) -> None:
        if self.healthy:
            self.scheduler.fail("cancelled")
            self._in_flight = None          # what a queued step samples belongs to nobody any more
            self._emit_finished()
            self.healthy = False
