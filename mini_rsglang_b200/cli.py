"""Command line in the manner of the reference's `mini-rsglang` binary
(crates/server/src/main.rs:15-246): the same global options with the same defaults and
meanings where the engine has the thing they set, and its `generate` subcommand with the
same sampling options.  Prompts are token ids (`--token-ids 1,2,3`); there is no tokenizer,
so `--prompt`, `--chat` and `--enable-thinking` are not offered, and neither are `serve`
(no server) and the tensor-parallel options (one GPU).  `bench` is the reference's closed-loop
load test (main.rs:94-113, 266-300) with seeded random prompts; `--cache-mode` takes only
`cold`, because nothing is shared between requests here.  Added: `--dtype`, `--num-pages`,
`--token-ids-file` (several requests at once), and `random-model`, which writes a model
folder from a config.json and a seed."""
from __future__ import annotations

import argparse
import json
import sys

from .config.runtime_config import RuntimeConfig
from .errors import EngineError, InvalidRequest
from .sampling.params import SamplingParams


def parse_token_ids(text: str) -> list[int]:
    try:
        ids = [int(v.strip()) for v in text.split(",")]
    except ValueError:
        raise InvalidRequest("token_ids must be comma-separated integers") from None
    if any(i < 0 for i in ids):
        raise InvalidRequest("token_ids must be comma-separated integers")
    return ids


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(prog="mini-rsglang", description="B200-native LLM inference on one GPU")
    p.add_argument("--model", default="/models/store/Qwen/Qwen3-0.6B", help="folder with config.json and weights")
    p.add_argument("--device", type=int, default=0)
    p.add_argument("--kv-mib", type=int, default=2048, help="memory of the KV cache in MiB")
    p.add_argument("--max-seq-len", type=int, default=4096)
    p.add_argument("--page-size", type=int, default=16)
    p.add_argument("--prefill-budget", type=int, default=512)
    p.add_argument("--max-running", type=int, default=32)
    p.add_argument("--max-waiting", type=int, default=256)
    p.add_argument("--no-prefix-cache", action="store_true",
                   help="do not share the cache pages of equal first tokens between requests")
    p.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    p.add_argument("--num-pages", type=int, default=None, help="size of the page pool (overrides --kv-mib)")
    p.add_argument("--random-weights", type=int, default=None, metavar="SEED",
                   help="take only config.json from --model and draw the weights on the device from this seed "
                        "(other tensors than `random-model` writes for the seed: those are drawn on the CPU)")
    sub = p.add_subparsers(dest="command", required=True)

    g = sub.add_parser("generate", help="generate from token ids")
    g.add_argument("--token-ids", help="comma-separated token ids of one prompt")
    g.add_argument("--token-ids-file", help="file with one comma-separated prompt per line")
    g.add_argument("--json", action="store_true", help="print every event as one JSON line")
    g.add_argument("--max-tokens", type=int, default=128)
    g.add_argument("--temperature", type=float, default=0.0)
    g.add_argument("--top-k", type=int, default=None)
    g.add_argument("--top-p", type=float, default=1.0)
    g.add_argument("--seed", type=int, default=0)
    g.add_argument("--ignore-eos", action="store_true")

    b = sub.add_parser("bench", help="closed-loop load test: fixed prompt and output lengths, fixed concurrency")
    b.add_argument("--input-tokens", type=int, default=128)
    b.add_argument("--output-tokens", type=int, default=32)
    b.add_argument("--requests", type=int, default=16)
    b.add_argument("--concurrency", type=int, default=8)
    b.add_argument("--cache-mode", choices=["cold", "hot", "both"], default="cold")
    b.add_argument("--output", help="also write the report to this file")
    b.add_argument("--seed", type=int, default=0, help="seed of the random prompts")

    r = sub.add_parser("random-model", help="write a model folder with seeded random weights")
    r.add_argument("--config", required=True, help="a config.json to take the sizes from")
    r.add_argument("--seed", type=int, required=True)
    r.add_argument("--out", required=True)
    r.add_argument("--weights-dtype", choices=["bfloat16", "float32"], default="bfloat16")
    return p


def runtime_config(args) -> RuntimeConfig:
    return RuntimeConfig(max_seq_len=args.max_seq_len, page_size=args.page_size, prefill_budget=args.prefill_budget,
                         max_running=args.max_running, max_waiting=args.max_waiting,
                         prefix_cache=not args.no_prefix_cache)


def load_engine(args, limits: RuntimeConfig):
    """The engine of the command line: weights from the model folder, or, with --random-weights, seeded random ones
    for the folder's config.json, drawn on the device."""
    from .engine.handle import EngineHandle

    if args.random_weights is None:
        return EngineHandle.load(args.model, args.device, args.kv_mib * 1024 * 1024, limits, dtype=args.dtype,
                                 num_pages=args.num_pages)
    from .models.registry import load_config

    return EngineHandle.from_random(load_config(args.model), args.random_weights, args.device, args.kv_mib * 1024 * 1024,
                                    limits, dtype=args.dtype, num_pages=args.num_pages)


def event_json(event) -> str:
    """One event in the reference's JSON shape (serde's externally tagged enum)."""
    from .engine.handle import Error, Finished, Token

    if isinstance(event, Token):
        return json.dumps({"Token": {"request_id": event.request_id, "token_id": event.token_id, "text": ""}})
    if isinstance(event, Finished):
        return json.dumps({"Finished": {"request_id": event.request_id, "reason": event.reason,
                                        "prompt_tokens": event.prompt_tokens,
                                        "completion_tokens": event.completion_tokens,
                                        "cached_tokens": event.cached_tokens}})
    if isinstance(event, Error):
        return json.dumps({"Error": {"request_id": event.request_id, "message": event.message}})
    raise TypeError(event)


def command_generate(args) -> int:
    from .engine.handle import EngineHandle, Error, Finished, GenerateRequest, Token, TokenIds

    if bool(args.token_ids) == bool(args.token_ids_file):
        raise InvalidRequest("give exactly one of --token-ids and --token-ids-file")
    if args.token_ids:
        prompts = [parse_token_ids(args.token_ids)]
    else:
        with open(args.token_ids_file) as f:
            prompts = [parse_token_ids(line) for line in f if line.strip()]
    sampling = SamplingParams(temperature=args.temperature, top_k=args.top_k, top_p=args.top_p, seed=args.seed,
                              max_tokens=args.max_tokens, ignore_eos=args.ignore_eos)
    sampling.validate()
    if args.kv_mib <= 0:
        raise InvalidRequest("kv_mib must be positive")
    engine = load_engine(args, runtime_config(args))
    streams = [engine.generate(GenerateRequest(TokenIds(p), sampling)) for p in prompts]
    completed = True
    for stream in streams:
        tokens = []
        for event in stream:
            if args.json:
                print(event_json(event), flush=True)
            if isinstance(event, Token):
                tokens.append(event.token_id)
            elif isinstance(event, Error):
                raise EngineError(event.message)
            elif isinstance(event, Finished):
                if not args.json:
                    print(",".join(str(t) for t in tokens), flush=True)
                    print(f"{event.reason.capitalize()}: prompt={event.prompt_tokens}, "
                          f"generated={event.completion_tokens}, cached={event.cached_tokens}", file=sys.stderr)
                completed = completed and event.reason in ("stop", "length")
    engine.shutdown()
    if not completed:
        raise EngineError("generation did not complete")
    return 0


def command_bench(args) -> int:
    from .engine import load_test
    from .engine.handle import EngineHandle

    if args.kv_mib <= 0:
        raise InvalidRequest("kv_mib must be positive")
    runs = []
    for warm in {"cold": (False,), "hot": (True,), "both": (False, True)}[args.cache_mode]:
        limits = runtime_config(args)
        limits.prefix_cache = warm          # a cold run shares nothing, a hot one reads a prompt that is in the cache
        engine = load_engine(args, limits)
        try:
            runs.append(load_test.run(engine, args.input_tokens, args.output_tokens, args.requests, args.concurrency,
                                      args.seed, warm=warm))
        finally:
            engine.shutdown()
    report = json.dumps({"backend": "b200-tcgen05-tma", "devices": [args.device], "runs": runs}, indent=2)
    if args.output:
        with open(args.output, "w") as f:
            f.write(report)
    print(report)
    return 0


def command_random_model(args) -> int:
    import torch

    from .models.registry import config_from_dict
    from .weights.random_init import write_random_model

    with open(args.config) as f:
        config = config_from_dict(json.load(f))
    dtype = torch.bfloat16 if args.weights_dtype == "bfloat16" else torch.float32
    write_random_model(args.out, config, args.seed, dtype)
    print(args.out)
    return 0


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    try:
        if args.command == "generate":
            return command_generate(args)
        if args.command == "bench":
            return command_bench(args)
        return command_random_model(args)
    except EngineError as e:
        print(f"error: {type(e).__name__}: {e}", file=sys.stderr)
        return 1
