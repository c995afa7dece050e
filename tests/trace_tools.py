"""Helpers of the replay tests: traces in the replay program's input format for the four ways
of cutting the same requests, a driver for `bin/trace_run`, and the comparison gates."""
from __future__ import annotations

import json
import os
import random
import subprocess
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TRACE_RUN = os.path.join(ROOT, "bin", "trace_run")


def requests_for(vocab: int, lengths, seed: int) -> dict[str, list[int]]:
    rng = random.Random(seed)
    return {f"r{i}": [rng.randrange(vocab) for _ in range(n)] for i, n in enumerate(lengths)}


def rounded(n: int, unit: int = 64) -> int:
    return -(-n // unit) * unit


class Trace:
    """Steps in the input format, and for every step which (request, position) each row is."""

    def __init__(self):
        self.steps: list[dict] = []
        self.rows: list[list[tuple[str, int]]] = []

    def add(self, entries: list[tuple[str, int, list[int], list[int]]], end=()):
        """entries: (request, start position, tokens, wanted places among them)."""
        self.steps.append({"step": len(self.steps),
                           "entries": [{"id": r, "tokens": t, "want": w} for r, _, t, w in entries],
                           "end": list(end)})
        self.rows.append([(r, s + w) for r, s, _, ws in entries for w in ws])


def trace_whole(reqs) -> Trace:
    """Each request alone and whole, every position wanted."""
    t = Trace()
    for name, tokens in reqs.items():
        t.add([(name, 0, tokens, list(range(len(tokens))))], end=[name])
    return t


def trace_decode_tail(reqs, tail: int = 32) -> Trace:
    """Most of a request in one step, then its last `tail` tokens one by one."""
    t = Trace()
    for name, tokens in reqs.items():
        head = max(len(tokens) - tail, 1)
        t.add([(name, 0, tokens[:head], [head - 1])])
        for p in range(head, len(tokens)):
            t.add([(name, p, [tokens[p]], [0])], end=[name] if p == len(tokens) - 1 else [])
        if head == len(tokens):
            t.add([], end=[name])
    return t


def trace_portions(reqs, seed: int) -> Trace:
    """Portions of changing size, down to two tokens; first, last and a middle place wanted."""
    rng = random.Random(seed)
    t = Trace()
    for name, tokens in reqs.items():
        p = 0
        while p < len(tokens):
            n = min(rng.choice([2, 2, 3, 5, 7, 13, 16, 17, 31, 33]), len(tokens) - p)
            want = sorted({0, n // 2, n - 1})
            t.add([(name, p, tokens[p:p + n], want)], end=[name] if p + n == len(tokens) else [])
            p += n
    return t


def trace_mixed(reqs, seed: int, max_live: int = 4, tail: int = 32) -> tuple[Trace, int]:
    """Up to `max_live` requests at a time: portions of some beside single decoded tokens of
    others; a request leaves when it is done and the next one takes over its pages.  Also
    returns the pool size (tokens) that the live requests need at most, each rounded up to 64."""
    rng = random.Random(seed)
    t = Trace()
    queue = list(reqs.items())
    live: dict[str, int] = {}          # request -> tokens already fed
    peak = 0
    while queue or live:
        while queue and len(live) < max_live:
            name, _ = queue.pop(0)
            live[name] = 0
        peak = max(peak, sum(rounded(len(reqs[n])) for n in live))
        entries, ending = [], []
        for name in list(live):
            if len(live) > 1 and rng.random() < 0.2:
                continue                   # a request may sit a step out
            tokens, p = reqs[name], live[name]
            in_tail = p >= max(len(tokens) - tail, 1)
            n = 1 if in_tail else min(rng.choice([2, 3, 5, 8, 11, 16, 19]), max(len(tokens) - tail, 1) - p)
            entries.append((name, p, tokens[p:p + n], [n - 1] if rng.random() < 0.8 or in_tail else []))
            live[name] = p + n
            if p + n == len(tokens):
                ending.append(name)
                del live[name]
        if entries or ending:
            t.add(entries, end=ending)
    return t, peak


class TraceRun:
    """Drives one `bin/trace_run` process: a step is written only after the `done` of the last."""

    def __init__(self, model: str, dtype: str, out: str, max_tokens: int, env=None, extra=()):
        self.out = out
        self.proc = subprocess.Popen(
            [sys.executable, TRACE_RUN, "--model", model, "--dtype", dtype, "--out", out, "--max-tokens", str(max_tokens),
             *extra], stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, env=env)

    def step(self, record: dict, vocab: int):
        self.proc.stdin.write(json.dumps(record) + "\n")
        self.proc.stdin.flush()
        line = self.proc.stdout.readline().strip()
        assert line == f"done {record['step']}", f"trace_run answered {line!r} to step {record['step']}"
        wanted = sum(len(e["want"]) for e in record["entries"])
        path = os.path.join(self.out, f"{record['step']}.f32")
        if wanted == 0:
            assert not os.path.exists(path)
            return None
        data = np.fromfile(path, dtype="<f4")
        assert data.size == wanted * vocab, f"step {record['step']}: {data.size} floats for {wanted} rows"
        os.remove(path)
        return torch.from_numpy(data.reshape(wanted, vocab).astype(np.float64))

    def close(self) -> int:
        self.proc.stdin.close()
        return self.proc.wait(timeout=120)


def renumber(trace: Trace, first: int, prefix: str) -> Trace:
    """The same trace with step numbers from `first` and request ids of its own."""
    out = Trace()
    for step, rows in zip(trace.steps, trace.rows):
        out.steps.append({"step": first + step["step"],
                          "entries": [dict(e, id=prefix + e["id"]) for e in step["entries"]],
                          "end": [prefix + n for n in step["end"]]})
        out.rows.append(rows)
    return out


def sharpen(folder, out, factor):
    """The same model with q and k head-norm weights scaled: attention gets peaked, so a key
    read from the wrong place moves the logits by far more than rounding."""
    from safetensors.torch import load_file
    from mini_rsglang_b200.weights import write_safetensors
    tensors = load_file(os.path.join(folder, "model.safetensors"))
    for name in tensors:
        if name.endswith("q_norm.weight") or name.endswith("k_norm.weight"):
            tensors[name] = (tensors[name].float() * factor).to(tensors[name].dtype)
    os.makedirs(out, exist_ok=True)
    write_safetensors(os.path.join(out, "model.safetensors"), tensors)
    with open(os.path.join(folder, "config.json")) as f, open(os.path.join(out, "config.json"), "w") as g:
        g.write(f.read())
    return out


# ------------------------------------------------------------------------------ gates
# 32-bit path against the exact (float64) plain implementation: the engine sums in float32, so
# a logit differs by rounding of order 1e-6 of the row's scale; 2e-5 leaves room for long sums.
F32_REL = 2e-5
# bfloat16 path: the reference's own gate for a bfloat16 engine against a reference model
# (scripts/verify_model.py:158-170): NRMSE <= 0.02 and cosine >= 0.999, per row.
BF16_NRMSE, BF16_COSINE = 0.02, 0.999


def check_rows(got: torch.Tensor, want: torch.Tensor, dtype: str, what: str) -> None:
    assert got.shape == want.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(want.shape)}"
    assert torch.isfinite(got).all(), f"{what}: non-finite logits"
    for i in range(got.shape[0]):
        g, w = got[i], want[i]
        if dtype == "float32":
            err, scale = (g - w).abs().max().item(), max(1.0, w.abs().max().item())
            assert err <= F32_REL * scale, f"{what} row {i}: max error {err:.3e} over scale {scale:.3f}"
        else:
            nrmse = ((g - w).pow(2).mean().sqrt() / w.pow(2).mean().sqrt()).item()
            cosine = torch.nn.functional.cosine_similarity(g, w, dim=0).item()
            assert nrmse <= BF16_NRMSE and cosine >= BF16_COSINE, f"{what} row {i}: NRMSE {nrmse:.4f}, cosine {cosine:.5f}"
