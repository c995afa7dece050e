"""Trace replay: feeds given token ids through the model step by step and writes logits.

It samples nothing and has no model code of its own: it opens requests in the engine's cache
manager, extends them by each step's tokens, runs the engine's step function and closes the
requests a step names as finished.  The reference's counterpart is its `forward` example
(crates/engine/examples/forward.rs:12-127: teacher-forced batches, one file of float32 logits
per case and step).

Input, one JSON object a line:
    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}
For a step in which something is wanted, `<out>/<step>.f32` holds the logits at the wanted
places, in the order of the entries and of `want`, little-endian float32 [wanted, vocab].
After every step a line `done <step>` is printed and flushed.

`--observe ID` also writes, for every step that brings tokens of request ID, what the reference's
observer sees layer by layer (crates/models/src/qwen3.rs:159-229; its `trace` example,
crates/engine/examples/trace.rs): `<out>/observe/<step>.<label>.f32`, float32 [the request's tokens of the
step, width], labels `embedding`, `layerN-input_norm`, `-q_proj`, `-q_norm`, `-q_rope`, `-k_rope`,
`-v_proj`, `-attn`, `-swiglu`, `-output`, `final_norm`."""
from __future__ import annotations

import argparse
import json
import os
import sys

import numpy as np

from ..config.runtime_config import RuntimeConfig
from ..errors import EngineError, InvalidRequest
from ..models.registry import load_config
from .runner import ModelRunner, SequenceStep

MAX_LIVE = 8      # state slots; a trace holds up to four live requests


class Replayer:
    def __init__(self, model: str, dtype: str, max_tokens: int, device: str = "cuda:0", page_size: int = 16,
                 observe: str | None = None):
        config = load_config(model)
        pages = -(-int(max_tokens) // page_size)
        limits = RuntimeConfig(max_seq_len=min(config.max_position_embeddings, max(pages * page_size, page_size)),
                               page_size=page_size, prefill_budget=max(pages * page_size, 1), max_running=MAX_LIVE)
        self.runner = ModelRunner.load(model, dtype=dtype, device=device, limits=limits, num_pages=pages)
        self.observed = observe            # the request whose layers are written out, or None
        self.seen: dict[str, np.ndarray] = {}
        self.ids: dict[str, int] = {}
        self.lengths: dict[str, int] = {}
        self.next_id = 1

    def step(self, record: dict):
        """Runs one step; returns the logits [wanted, vocab] as a float32 array, or None."""
        cache = self.runner.cache
        batch = []
        for entry in record.get("entries", []):
            name = str(entry["id"])
            tokens = [int(t) for t in entry["tokens"]]
            if name not in self.ids:
                self.ids[name] = self.next_id
                self.next_id += 1
                self.lengths[name] = 0
                cache.open(self.ids[name])
            start = self.lengths[name]
            cache.extend(self.ids[name], start + len(tokens))
            batch.append(SequenceStep(self.ids[name], tokens, start, [int(w) for w in entry.get("want", [])]))
        logits = None
        self.seen = {}
        observe = None
        names = [str(entry["id"]) for entry in record.get("entries", [])]
        if self.observed is not None and self.observed in names:
            at = names.index(self.observed)
            first = sum(len(seq.tokens) for seq in batch[:at])
            rows = slice(first, first + len(batch[at].tokens))

            def observe(label, tensor):
                self.seen[label] = tensor[rows].float().cpu().numpy().astype("<f4")
        if batch:
            logits = self.runner.step(batch, observe)
            for seq in batch:
                cache.trim(seq.request_id, seq.start_pos + len(seq.tokens))
            for entry, seq in zip(record["entries"], batch):
                self.lengths[str(entry["id"])] = seq.start_pos + len(seq.tokens)
        for name in record.get("end", []):
            name = str(name)
            if name not in self.ids:
                raise InvalidRequest(f"step {record.get('step')}: cannot end unknown request {name!r}")
            cache.close(self.ids.pop(name))
            del self.lengths[name]
        return None if logits is None else logits.float().cpu().numpy().astype("<f4")


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    parser.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    parser.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    parser.add_argument("--out", required=True, help="folder for <step>.f32 files")
    parser.add_argument("--max-tokens", type=int, required=True,
                        help="most tokens that live requests hold at any time; the cache pool is made for this many")
    parser.add_argument("--device", default="cuda:0")
    parser.add_argument("--page-size", type=int, default=16,
                        help="tokens of a cache page (a power of two); --max-tokens is rounded up to whole pages")
    parser.add_argument("--observe", metavar="ID", help="also write the layers of this request, step by step, to <out>/observe/")
    args = parser.parse_args(argv)
    os.makedirs(args.out, exist_ok=True)
    if args.observe is not None:
        os.makedirs(os.path.join(args.out, "observe"), exist_ok=True)
    try:
        replayer = Replayer(args.model, args.dtype, args.max_tokens, args.device, page_size=args.page_size, observe=args.observe)
        for line in sys.stdin:
            line = line.strip()
            if not line:
                continue
            record = json.loads(line)
            logits = replayer.step(record)
            if logits is not None:
                logits.tofile(os.path.join(args.out, f"{record['step']}.f32"))
            for label, rows in replayer.seen.items():
                rows.tofile(os.path.join(args.out, "observe", f"{record['step']}.{label}.f32"))
            print(f"done {record['step']}", flush=True)
    except EngineError as e:
        print(f"trace_run: {type(e).__name__}: {e}", file=sys.stderr, flush=True)
        return 1
    return 0
