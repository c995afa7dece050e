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
from .scheduler import Scheduler


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
        """Plans, runs and commits one step.  False when there was nothing to run."""
        if not self.healthy:
            raise EngineStopped("engine stopped")
        plan = self.scheduler.plan()
        self._emit_finished()
        if not plan:
            return False
        batch = [SequenceStep(p.request_id, p.tokens, p.start_pos, [len(p.tokens) - 1] if p.sample else [])
                 for p in plan]
        sampled_ids = [p.request_id for p in plan if p.sample]
        try:
            logits = self.runner.forward(batch)
            if sampled_ids:
                tokens = self.sampler.sample(logits, [self.params[i] for i in sampled_ids],
                                             [self.generated[i] for i in sampled_ids])
            else:
                tokens = []
                torch.cuda.current_stream().synchronize()
            kernels.check_device_errors()
        except (EngineError, RuntimeError) as e:
            # a failed step ends every request and gives every page back (scheduler.rs:332-359)
            self.healthy = False
            message = f"{type(e).__name__}: {e}"
            for stream in list(self.streams.values()):
                stream.events.append(Error(stream.request_id, message))
            self.scheduler.fail("error")
            self._emit_finished()
            raise BackendError(message) from e
        self.scheduler.commit(tokens)
        for request_id, token in zip(sampled_ids, tokens):
            self.generated[request_id] += 1
            stream = self.streams.get(request_id)
            if stream is not None:
                stream.events.append(Token(request_id, token))
        self._emit_finished()
        return True

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
            self._emit_finished()
            self.healthy = False
