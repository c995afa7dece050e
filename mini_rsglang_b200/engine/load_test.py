"""A closed-loop load test of the engine: a fixed number of requests, a fixed number of them
in flight, fixed prompt and output lengths (reference: `mini-rsglang bench`,
crates/server/src/bench.rs:16-170).  The reference tokenises a repeated sentence; without a
tokenizer the prompts here are seeded uniform random token ids of the same length.  Cold
(`warm=False`): every request's prompt is different and the engine shares nothing.  Warm: as in
the reference every request brings the same prompt to an engine that shares prefixes, after one
request of one token that leaves the prompt's pages behind (bench.rs:41-49).

The warm-up waves (two, as in the reference, bench.rs:50) run the measured workload itself, all its
requests at its concurrency, not only one batch of `concurrency` prompts: this engine records a step's
shape at its first use, and the shapes of the steady state (requests that finish while others decode
and new ones arrive) do not occur in a single batch.  Measured at the 0.6B shape, 16 requests, 8 in
flight, 128 prompt and 32 generated tokens: time to the first token p50 23 ms with single batches as
warm-up (new shapes are recorded under the clock), 3.2 ms with the workload."""
from __future__ import annotations

import math
import random
import time

from ..errors import BackendError, InvalidRequest
from ..sampling.params import SamplingParams
from .handle import EngineHandle, Error, Finished, GenerateRequest, Token, TokenIds


def percentile(values: list[float], p: float) -> float:
    """The reference's percentile: the element at round((n - 1) * p) of the sorted values, halves away from zero."""
    if not values:
        return 0.0
    ordered = sorted(values)
    return ordered[int(math.floor((len(ordered) - 1) * p + 0.5))]


def _wave(engine: EngineHandle, prompts: list[list[int]], output_tokens: int, concurrency: int):
    """Runs the prompts with at most `concurrency` in flight; returns per request the time to the first
    token, the gaps between tokens and the whole latency (seconds)."""
    sampling = SamplingParams(max_tokens=output_tokens, ignore_eos=True)
    pending = list(prompts)
    live: dict[int, dict] = {}
    first, gaps, latency = [], [], []
    while pending or live:
        while pending and len(live) < concurrency:
            stream = engine.generate(GenerateRequest(TokenIds(pending.pop(0)), sampling))
            live[stream.request_id] = {"stream": stream, "start": time.perf_counter(), "last": None, "tokens": 0}
        if not engine.run_step() and not any(state["stream"].events for state in live.values()):
            raise BackendError("scheduler is idle but requests are unfinished")
        now = time.perf_counter()
        for request_id in list(live):
            state = live[request_id]
            while state["stream"].events:
                event = state["stream"].events.popleft()
                if isinstance(event, Token):
                    if state["last"] is None:
                        first.append(now - state["start"])
                    else:
                        gaps.append(now - state["last"])
                    state["last"] = now
                    state["tokens"] += 1
                elif isinstance(event, Error):
                    raise BackendError(event.message)
                elif isinstance(event, Finished):
                    if event.reason != "length" or state["tokens"] != output_tokens:
                        raise BackendError("benchmark did not generate fixed output length")
                    latency.append(now - state["start"])
                    del live[request_id]
                    break
    return first, gaps, latency


def run(engine: EngineHandle, input_tokens: int, output_tokens: int, requests: int, concurrency: int,
        seed: int = 0, warmup_waves: int = 2, warm: bool = False) -> dict:
    if min(input_tokens, output_tokens, requests, concurrency) <= 0 or concurrency > engine.config.max_running:
        raise InvalidRequest("positive benchmark sizes required; concurrency must be <= max_running")
    rng = random.Random(seed)
    vocab = engine.info["vocab_size"]

    shared_prompt = [rng.randrange(vocab) for _ in range(input_tokens)]

    def prompts(n):
        if warm:
            return [list(shared_prompt) for _ in range(n)]
        return [[rng.randrange(vocab) for _ in range(input_tokens)] for _ in range(n)]

    if warm:
        if not engine.config.prefix_cache:
            raise InvalidRequest("a warm run needs an engine that shares prefixes")
        engine.generate_many([shared_prompt], SamplingParams(max_tokens=1, ignore_eos=True))
    for _ in range(warmup_waves):          # the measured batch and token shapes, before the clock starts
        _wave(engine, prompts(requests), output_tokens, concurrency)
    before = engine.metrics()
    started = time.perf_counter()
    first, gaps, latency = _wave(engine, prompts(requests), output_tokens, concurrency)
    elapsed = time.perf_counter() - started

    def spread(values):
        return {"p50": percentile(values, 0.5) * 1000.0, "p95": percentile(values, 0.95) * 1000.0}

    after = engine.metrics()
    return {"warmup_waves": warmup_waves, "cache_mode": "warm_prefix" if warm else "disabled", "model": engine.info["model_id"],
            "input_tokens": input_tokens, "output_tokens": output_tokens, "requests": requests, "concurrency": concurrency,
            "elapsed_s": elapsed, "output_tokens_per_s": requests * output_tokens / elapsed,
            "requests_per_s": requests / elapsed, "ttft_ms": spread(first), "itl_ms": spread(gaps),
            "latency_ms": spread(latency), "raw_ttft_s": first, "raw_itl_s": gaps, "raw_latency_s": latency,
            "cached_tokens": after["cached_tokens"] - before["cached_tokens"], "peak_memory_bytes": after["peak_memory_bytes"], "metrics": after}
