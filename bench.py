"""Benchmark of the engine on one B200: decode tokens a second at the Qwen3-8B shape.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]
    python bench.py --shape 14b --batch 16 --context 8192        decode at the Qwen3-14B shape
    python bench.py --shape 0.6b --continuous                    continuous batching at the Qwen3-0.6B shape

A "step" is one decode step: every live request gets its next token.  The default run has the
layer sizes of the Qwen3-8B shape with seeded random weights (bfloat16), a batch of 8 and a
context of 4,096 tokens: the timed steps are the last K before each request reaches 4,096
tokens.  One JSON line is printed:
  value      decoded tokens a second, timed on the device with CUDA events around the K steps
             (synthetic token ids, next token chosen by the arg-max kernel on the device);
  e2e        the same through the Python entry point (`EngineHandle`): every step copies the
             step's token ids from pinned host memory and reads the sampled tokens back;
  prefill    one prompt of 2,048 tokens in one step, with its fraction of the bf16 peak;
  roofline   bytes a decode step must read (every weight once and the live requests' cache)
             divided by its time, against the measured copy bandwidth;
  points     decode at batch 1 and batch 64, each with the same fraction of the copy bandwidth.
  prefill also carries `chunked_4x512_ms`: the same prompt in four steps of 512 tokens.
`--shape 14b` (40 layers, width 5120, 40 / 8 heads, feed-forward 17408) and `--shape 0.6b` (28 layers, width 1024,
16 / 8 heads, feed-forward 3072, tied head) run the same measurement at those sizes, with `--batch` and `--context`.
`--continuous` is the serving workload: 64 requests with seeded prompt lengths uniform in 16 to 2,048 tokens and 64
generated tokens each, through `EngineHandle` with prompts cut into portions under a budget of 512 tokens a step; its
line reports prompt and generated tokens a second, the mean step time and the share of steps that were replayed
from a recording.
Peaks come from MEASURED_PEAKS.json when the file exists.  The engine runs on one GPU; for
--gpus N > 1 a line says so and the exit code is 2.  The reference arm cannot run here (the
reference is a Rust workspace without a Python package, and supports no sm_100 device), so
`--impl reference` prints its `unavailable` line."""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

QWEN3_8B = dict(model_type="qwen3", architectures=["Qwen3ForCausalLM"], hidden_size=4096, intermediate_size=12288,
                num_hidden_layers=36, num_attention_heads=32, num_key_value_heads=8, head_dim=128, vocab_size=151936,
                max_position_embeddings=40960, rms_norm_eps=1e-6, rope_theta=1000000.0, tie_word_embeddings=False,
                hidden_act="silu", eos_token_id=151645)
QWEN3_06B = dict(QWEN3_8B, hidden_size=1024, intermediate_size=3072, num_hidden_layers=28, num_attention_heads=16,
                 num_key_value_heads=8, head_dim=128, tie_word_embeddings=True)
QWEN3_14B = dict(QWEN3_8B, hidden_size=5120, intermediate_size=17408, num_hidden_layers=40, num_attention_heads=40,
                 num_key_value_heads=8, head_dim=128)
SHAPES = {"8b": ("Qwen3-8B shape", QWEN3_8B), "0.6b": ("Qwen3-0.6B shape", QWEN3_06B), "14b": ("Qwen3-14B shape", QWEN3_14B)}
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def peaks() -> dict:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            data = json.load(f)
        return {"hbm_gbs": float(data["hbm_gbs"]), "bf16_tflops": float(data["bf16_tflops"]), "source": "measured"}
    return dict(FALLBACK_PEAKS)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        clocks, max_clock, reasons = [], None, set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in out.splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) != 6:
                continue
            try:
                clocks.append(float(parts[0]))
                max_clock = float(parts[1])
            except ValueError:
                continue
            for name, value in zip(names, parts[2:]):
                if value.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(clocks) if clocks else None, "sm_max_mhz": max_clock,
                "reasons": sorted(reasons), "samples": len(clocks)}


def model_numbers(cfg: dict, layers: int) -> dict:
    """Weight bytes a decode step reads, cache bytes per context token, flops per prompt token."""
    h, i, v = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    nq, nkv, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    per_layer = (nq + 2 * nkv) * d * h + h * nq * d + 2 * i * h + h * i
    return {"layer_params": per_layer, "head_params": v * h,
            "weight_bytes": 2 * (layers * per_layer + v * h),       # a tied head reads the embedding table: the same bytes
            "kv_bytes_per_token": layers * 2 * nkv * d * 2,
            "linear_flops_per_token": 2 * layers * per_layer,
            "attn_flops_per_pair": 4 * nq * d * layers}


def kernel_shares(torch, run) -> None:
    """Runs `run` under torch.profiler and prints, kernel by kernel, launches, the sum and the mean of their
    durations and the share of the sum (kernels that start under their predecessor overlap it, so the sum is more
    than the wall clock: compare shares)."""
    import collections

    from torch.profiler import ProfilerActivity, profile

    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        run()
        torch.cuda.synchronize()
    table = collections.defaultdict(lambda: [0, 0.0])
    for event in prof.events():
        if event.device_type.name == "CUDA":
            entry = table[event.name[:100]]
            entry[0] += 1
            entry[1] += event.device_time
    total = sum(t for _, t in table.values()) or 1.0
    print(f"kernels: {total / 1e3:.1f} ms in {sum(n for n, _ in table.values())} launches", file=sys.stderr)
    for name, (n, t) in sorted(table.items(), key=lambda kv: -kv[1][1])[:24]:
        print(f"{t / 1e3:9.2f} ms {100 * t / total:5.1f}% {n:7d} launches {t / n:8.1f} us  {name}", file=sys.stderr)


def continuous_run(args, torch, shape_name: str, cfg: dict, peak: dict) -> dict:
    """The serving workload of the 0.6B configuration: `--requests` requests (64) whose prompt lengths are drawn
    uniformly from 16 to 2,048 (seeded), `--output-tokens` generated tokens each (64), all submitted at once to
    `EngineHandle`; prompts are cut into portions under a budget of 512 tokens a step and run beside the decoded
    tokens of the requests that are further on.  A first wave of the same lengths (other tokens) runs untimed so
    that every kernel has been built and every step shape has been recorded once: the timed wave is the steady
    state of a server that has seen its traffic before."""
    import random

    from mini_rsglang_b200 import RuntimeConfig, SamplingParams
    from mini_rsglang_b200.engine import EngineHandle
    from mini_rsglang_b200.models import config_from_dict

    config = config_from_dict(cfg)
    requests, out_tokens, budget, page = args.requests, args.output_tokens, args.prefill_budget, 16
    rng = random.Random(20240611)
    lengths = [rng.randint(16, 2048) for _ in range(requests)]
    max_running = min(requests, args.max_running)
    max_seq_len = 2048 + out_tokens
    pages = max_running * (-(-max_seq_len // page) + 1) + 8
    limits = RuntimeConfig(max_seq_len=max_seq_len, page_size=page, prefill_budget=budget, max_running=max_running,
                           max_waiting=max(256, requests))
    engine = EngineHandle.from_random(config, seed=1, dtype="bfloat16", config=limits, num_pages=pages)
    runner = engine.runner
    params = SamplingParams(max_tokens=out_tokens, ignore_eos=True)

    def prompts(ns):
        return [[rng.randrange(cfg["vocab_size"]) for _ in range(n)] for n in ns]

    engine.generate_many(prompts(lengths), params)     # warm-up wave of the same lengths, untimed: every step shape is recorded
    work = prompts(lengths)
    torch.cuda.synchronize()
    steps0, recorded0, h2d0 = runner.steps, runner.recorded_steps, runner.h2d_bytes
    sampler = ClockSampler()
    sampler.start()
    t0 = time.perf_counter()
    results = engine.generate_many(work, params)
    torch.cuda.synchronize()
    elapsed = time.perf_counter() - t0
    clocks = sampler.stop()
    steps = runner.steps - steps0
    generated = sum(r.completion_tokens for r in results)
    prompt_tokens = sum(lengths)
    assert all(r.finish_reason == "length" and r.completion_tokens == out_tokens for r in results)
    recorded, h2d = runner.recorded_steps - recorded0, runner.h2d_bytes - h2d0
    if args.kernel_shares:
        kernel_shares(torch, lambda: engine.generate_many(prompts(lengths), params))
    engine.shutdown()
    total = prompt_tokens + generated
    return {
        "metric": f"continuous batching tok/s, {requests} requests of 16-2048 prompt tokens, {out_tokens} generated each ({shape_name})",
        "value": round(total / elapsed, 1), "unit": "tokens/s (prompt + generated)", "n_gpus": 1, "steps": steps, "warmup": 1,
        "ms_per_step": round(elapsed / steps * 1e3, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: seeded random weights, seeded prompt lengths, uniform random token ids",
        "prompt_tokens_per_s": round(prompt_tokens / elapsed, 1), "generated_tokens_per_s": round(generated / elapsed, 1),
        "prompt_tokens": prompt_tokens, "generated_tokens": generated, "elapsed_s": round(elapsed, 4),
        "recorded_step_share": round(recorded / max(steps, 1), 4),
        "h2d_bytes_per_step": h2d // max(steps, 1),
        "config": {"model": shape_name, "layers": cfg["num_hidden_layers"], "layers_of_shape": cfg["num_hidden_layers"],
                   "hidden": cfg["hidden_size"], "q_heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
                   "head_dim": cfg["head_dim"], "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"],
                   "tied_head": cfg["tie_word_embeddings"], "requests": requests, "max_running": max_running,
                   "prefill_budget": budget, "output_tokens": out_tokens, "page_size": page, "parallelism": "single GPU",
                   "timing": "wall clock around EngineHandle.generate_many, host tokens in and out", "peaks": peak["source"]},
        "clocks": clocks, "impl": "ours"}


def main() -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=64)
    parser.add_argument("--warmup", type=int, default=8)
    parser.add_argument("--impl", choices=["ours", "reference"], default="ours")
    parser.add_argument("--shape", choices=sorted(SHAPES), default="8b", help="layer sizes: Qwen3-8B (the default line), 0.6B or 14B")
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--context", type=int, default=4096)
    parser.add_argument("--layers", type=int, default=0, help="fewer layers than the shape has (named in config); 0: all of them")
    parser.add_argument("--no-points", action="store_true", help="skip the batch-1 and batch-64 points")
    parser.add_argument("--no-e2e", action="store_true")
    parser.add_argument("--continuous", action="store_true", help="the continuous-batching workload instead of the decode measurement")
    parser.add_argument("--requests", type=int, default=64, help="--continuous: requests")
    parser.add_argument("--output-tokens", type=int, default=64, help="--continuous: generated tokens a request")
    parser.add_argument("--prefill-budget", type=int, default=512, help="--continuous: tokens a step")
    parser.add_argument("--max-running", type=int, default=64, help="--continuous: requests in flight at most")
    parser.add_argument("--kernel-shares", action="store_true",
                        help="--continuous: after the timed wave, one more wave under torch.profiler; its kernels' shares of the "
                             "device's time go to standard error (not a timing)")
    args = parser.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference is a Rust workspace (no setup.py/pyproject.toml: pip cannot install it, "
                          "no cargo in the image) and its CUDA backend accepts only sm_80..sm_90"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported (run with --gpus 1)")
        return 2
    if args.warmup < 3:
        args.warmup = 3

    import torch

    from mini_rsglang_b200 import RuntimeConfig, SamplingParams, kernels
    from mini_rsglang_b200.engine import EngineHandle, GenerateRequest, SequenceStep, TokenIds
    from mini_rsglang_b200.models import config_from_dict

    torch.cuda.set_device(0)
    shape_name, shape = SHAPES[args.shape]
    full_layers = shape["num_hidden_layers"]
    layers = args.layers or full_layers
    cfg = dict(shape, num_hidden_layers=layers)
    peak = peaks()
    if args.continuous:
        print(json.dumps(continuous_run(args, torch, shape_name, cfg, peak)))
        return 0
    config = config_from_dict(cfg)
    numbers = model_numbers(cfg, layers)
    context, batch = args.context, args.batch
    default_line = args.shape == "8b"
    point_batches = [] if args.no_points or not default_line else [1, 64]
    max_batch = max([batch] + point_batches)
    page = 16
    pages = max_batch * (-(-context // page)) + 2 * (-(-2048 // page)) + 8
    limits = RuntimeConfig(max_seq_len=max(context, 2048), page_size=page, prefill_budget=2048, max_running=max_batch, max_waiting=256)
    engine = EngineHandle.from_random(config, seed=1, dtype="bfloat16", config=limits, num_pages=pages)
    runner = engine.runner
    for entry in runner.storage.entries:      # cache contents do not change the timing; avoid all-zero keys anyway
        entry.k.normal_(0.0, 1.0)
        entry.v.normal_(0.0, 1.0)
    gen = torch.Generator().manual_seed(7)

    def random_tokens(n):
        return torch.randint(0, cfg["vocab_size"], (n,), generator=gen).tolist()

    def timed(fn, repeat):
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        for _ in range(repeat):
            fn()
        end.record()
        torch.cuda.synchronize()
        return start.elapsed_time(end)

    # ---------------------------------------------------------------- prefill of 2,048 tokens: in one step, and in four of 512
    prefill_tokens = 2048
    prompt = random_tokens(prefill_tokens)

    def prefill_once(request, portion):
        runner.cache.open(request)
        for at in range(0, prefill_tokens, portion):
            runner.cache.extend(request, at + portion)
            runner.forward([SequenceStep(request, prompt[at:at + portion], at, [portion - 1] if at + portion == prefill_tokens else [])])

    def prefill_median(portion, first_id):
        samples = []
        for trial in range(3 + 3):
            ms = timed(lambda: prefill_once(first_id + trial, portion), 1)
            runner.cache.close(first_id + trial)
            if trial >= 3:
                samples.append(ms)
        return statistics.median(samples)

    prefill_time = prefill_median(prefill_tokens, 10_000)
    chunked_time = prefill_median(512, 11_000)
    prefill_flops = (prefill_tokens * numbers["linear_flops_per_token"]
                     + numbers["attn_flops_per_pair"] * prefill_tokens * (prefill_tokens + 1) // 2
                     + 2 * numbers["head_params"])
    prefill = {"value": round(prefill_tokens / prefill_time * 1e3, 1), "tokens": prefill_tokens,
               "ms": round(prefill_time, 3), "frac": round(prefill_flops / (prefill_time * 1e-3) / (peak["bf16_tflops"] * 1e12), 4),
               "flops": prefill_flops, "peak_tflops": peak["bf16_tflops"], "chunked_4x512_ms": round(chunked_time, 3),
               "chunked_4x512_value": round(prefill_tokens / chunked_time * 1e3, 1)}

    # ---------------------------------------------------------------- decode, timed on the device
    def decode_run(b, steps, warmup, sample_clocks=False):
        """b requests whose context ends at `context` after warmup + steps decode steps."""
        start_len = context - (warmup + steps)
        ids = list(range(20_000 + 1000 * b, 20_000 + 1000 * b + b))
        for r in ids:
            runner.cache.open(r)
            runner.cache.extend(r, start_len)
        picked = torch.empty(b, dtype=torch.int32, device=runner.device)
        position = [start_len]

        def one_step():
            p = position[0]
            for r in ids:
                runner.cache.extend(r, p + 1)
            tokens = random_tokens(b)
            logits = runner.forward([SequenceStep(r, [t], p, [0]) for r, t in zip(ids, tokens)])
            kernels.argmax(logits, picked)
            position[0] = p + 1

        timed(one_step, warmup)
        sampler = ClockSampler()
        if sample_clocks:
            sampler.start()
        launches_before = kernels.launch_count
        ms = timed(one_step, steps)
        launches = kernels.launch_count - launches_before
        clocks = sampler.stop() if sample_clocks else None
        for r in ids:
            runner.cache.close(r)
        mean_context = context - steps / 2
        return {"ms_per_step": ms / steps, "tokens_per_s": b * steps / ms * 1e3, "launches": launches,
                "clocks": clocks, "mean_context": mean_context}

    main_run = decode_run(batch, args.steps, args.warmup, sample_clocks=True)
    step_bytes = numbers["weight_bytes"] + batch * main_run["mean_context"] * numbers["kv_bytes_per_token"]
    achieved = step_bytes / (main_run["ms_per_step"] * 1e-3) / 1e9
    roofline = {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak["hbm_gbs"], "unit": "GB/s",
                "frac": round(achieved / peak["hbm_gbs"], 4), "bytes_per_step": int(step_bytes)}
    points = {}
    for b in point_batches:
        run = decode_run(b, max(args.steps // 2, 8), args.warmup)
        points[f"decode_b{b}"] = round(run["tokens_per_s"], 1)
        point_bytes = numbers["weight_bytes"] + b * run["mean_context"] * numbers["kv_bytes_per_token"]
        points[f"decode_b{b}_hbm_frac"] = round(point_bytes / (run["ms_per_step"] * 1e-3) / 1e9 / peak["hbm_gbs"], 4)

    # ---------------------------------------------------------------- the same through the Python entry point
    e2e = None
    if not args.no_e2e:
        total = args.warmup + args.steps
        # every request must still be live when the timing ends: the first one decodes while the others'
        # prompts are still running, a step for every 2,048 prompt tokens of the batch
        slack = batch * context // limits.prefill_budget + 16
        prompt_len = context - total - slack
        params = SamplingParams(max_tokens=total + slack, ignore_eos=True)
        streams = [engine.generate(GenerateRequest(TokenIds(random_tokens(prompt_len)), params)) for _ in range(batch)]
        while engine.scheduler.waiting() or any(engine.generated.get(s.request_id, 0) == 0 for s in streams):
            if not engine.run_step():                        # prompts, untimed
                raise RuntimeError("the scheduler went idle before every request had its first token")
            if len(engine.generated) < batch:
                raise RuntimeError("a request finished before the timing began; raise the slack")
        for _ in range(args.warmup):
            engine.run_step()
        torch.cuda.synchronize()
        h2d_before, steps_before = runner.h2d_bytes, runner.steps
        made_before = sum(engine.generated.values())
        t0 = time.perf_counter()
        for _ in range(args.steps):
            engine.run_step()
        torch.cuda.synchronize()
        elapsed = time.perf_counter() - t0
        made = sum(engine.generated.values()) - made_before
        timed_steps = runner.steps - steps_before
        e2e = {"value": round(made / elapsed, 1), "unit": "tokens/s", "tokens": made,
               "h2d_bytes_per_step": (runner.h2d_bytes - h2d_before) // max(timed_steps, 1),
               "d2h_bytes_per_step": 4 * batch, "ms_per_step": round(elapsed / args.steps * 1e3, 3)}
        engine.shutdown()

    line = {
        "metric": f"decode tok/s at batch {batch}, context {context} ({shape_name})", "value": round(main_run["tokens_per_s"], 1),
        "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(main_run["ms_per_step"], 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic: seeded random weights, uniform random token ids",
        "config": {"model": shape_name, "layers": layers, "layers_of_shape": full_layers,
                   "hidden": cfg["hidden_size"], "q_heads": cfg["num_attention_heads"],
                   "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
                   "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"], "global_batch": batch,
                   "seq_len": context, "page_size": page, "parallelism": "single GPU",
                   "l2": "inputs larger than L2 (weights read every step)", "peaks": peak["source"]},
        "clocks": main_run["clocks"], "e2e": e2e, "gpu_launches": main_run["launches"],
        "prefill": prefill, "roofline": roofline, "points": points, "impl": "ours",
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
