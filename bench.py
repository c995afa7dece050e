"""Benchmark of the engine on one B200: decode tokens a second at the Qwen3-8B shape.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

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
FULL_LAYERS = 36
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
            "weight_bytes": 2 * (layers * per_layer + v * h),
            "kv_bytes_per_token": layers * 2 * nkv * d * 2,
            "linear_flops_per_token": 2 * layers * per_layer,
            "attn_flops_per_pair": 4 * nq * d * layers}


def main() -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=64)
    parser.add_argument("--warmup", type=int, default=8)
    parser.add_argument("--impl", choices=["ours", "reference"], default="ours")
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--context", type=int, default=4096)
    parser.add_argument("--layers", type=int, default=FULL_LAYERS, help="fewer layers than the 36 of the shape (named in config)")
    parser.add_argument("--no-points", action="store_true", help="skip the batch-1 and batch-64 points")
    parser.add_argument("--no-e2e", action="store_true")
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
    cfg = dict(QWEN3_8B, num_hidden_layers=args.layers)
    config = config_from_dict(cfg)
    numbers = model_numbers(cfg, args.layers)
    peak = peaks()
    context, batch = args.context, args.batch
    point_batches = [] if args.no_points else [1, 64]
    max_batch = max([batch] + point_batches)
    page = 16
    pages = max_batch * (-(-context // page)) + 2 * (-(-2048 // page)) + 8
    limits = RuntimeConfig(max_seq_len=context, page_size=page, prefill_budget=2048, max_running=max_batch, max_waiting=256)
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

    # ---------------------------------------------------------------- prefill of 2,048 tokens in one step
    prefill_tokens = 2048
    prompt = random_tokens(prefill_tokens)
    prefill_ms = []
    for trial in range(3 + 3):
        request = 10_000 + trial
        runner.cache.open(request)
        runner.cache.extend(request, prefill_tokens)
        ms = timed(lambda: runner.forward([SequenceStep(request, prompt, 0, [prefill_tokens - 1])]), 1)
        runner.cache.close(request)
        if trial >= 3:
            prefill_ms.append(ms)
    prefill_time = statistics.median(prefill_ms)
    prefill_flops = (prefill_tokens * numbers["linear_flops_per_token"]
                     + numbers["attn_flops_per_pair"] * prefill_tokens * (prefill_tokens + 1) // 2
                     + 2 * numbers["head_params"])
    prefill = {"value": round(prefill_tokens / prefill_time * 1e3, 1), "tokens": prefill_tokens,
               "ms": round(prefill_time, 3), "frac": round(prefill_flops / (prefill_time * 1e-3) / (peak["bf16_tflops"] * 1e12), 4),
               "flops": prefill_flops, "peak_tflops": peak["bf16_tflops"]}

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
        "metric": "decode tok/s at batch 8, context 4096 (Qwen3-8B shape)", "value": round(main_run["tokens_per_s"], 1),
        "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(main_run["ms_per_step"], 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic: seeded random weights, uniform random token ids",
        "config": {"model": "Qwen3-8B shape", "layers": args.layers, "layers_of_shape": FULL_LAYERS,
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
