"""Replay through `bin/trace_run`: the same requests whole, with the last 32 tokens decoded one
by one, in portions of changing size, and mixed with other requests in a pool so small that
pages are used again; in float32 and in bfloat16; each compared with the plain implementation."""
import functools

import pytest
import torch
from conftest import SHAPES

import plain_qwen3 as P
import trace_tools as T

pytestmark = pytest.mark.gpu

LENGTHS = {"A": [70, 45, 33, 100, 130, 64, 37, 90], "B": [1, 7, 17, 40, 129, 65, 96, 50], "C": [48, 80, 35, 66, 120],
           "D": [70, 45, 200, 33, 300, 131, 64], "R": [70, 45, 131, 64, 37]}
MODES = ("whole", "decode_tail", "portions", "mixed")


@functools.lru_cache(maxsize=None)
def plain_logits(folder: str, name: str):
    cfg, weights = P.PlainConfig.load(folder), P.load_plain_weights(folder)
    reqs = T.requests_for(cfg.vocab_size, LENGTHS[name], seed=100 + ord(name))
    return reqs, {r: P.logits_of_sequence(cfg, weights, tokens) for r, tokens in reqs.items()}


_results = {}


def replay(folder: str, name: str, dtype: str, tmp_path_factory):
    """All four traces of one configuration and dtype through one trace_run process."""
    key = (name, dtype)
    if key in _results:
        return _results[key]
    reqs, want = plain_logits(folder, name)
    vocab = SHAPES[name][0]["vocab_size"]
    mixed, peak = T.trace_mixed(reqs, seed=7)
    traces = {"whole": T.trace_whole(reqs), "decode_tail": T.trace_decode_tail(reqs),
              "portions": T.trace_portions(reqs, seed=5), "mixed": mixed}
    max_tokens = max(peak, max(T.rounded(len(t)) for t in reqs.values()))
    assert sum(T.rounded(len(t)) for t in reqs.values()) > max_tokens, "the pool must force pages to be used again"
    run = T.TraceRun(folder, dtype, str(tmp_path_factory.mktemp(f"out_{name}_{dtype}")), max_tokens)
    out = {}
    first = 0
    for mode in MODES:
        trace = T.renumber(traces[mode], first, f"{mode}-")
        first += len(trace.steps)
        rows = []
        for step, places in zip(trace.steps, trace.rows):
            got = run.step(step, vocab)
            if places:
                rows.append((step["step"], got, torch.stack([want[r][p] for r, p in places])))
        out[mode] = rows
    assert run.close() == 0
    _results[key] = out
    return out


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "R"])
def test_replay_matches_plain(request, model_folders, tmp_path_factory, name, dtype, mode):
    """"R": two layers of a real checkpoint's sizes, so that every cutting also runs at the sizes of production."""
    folder = request.getfixturevalue("real_size_folder") if name == "R" else model_folders[name]
    rows = replay(folder, name, dtype, tmp_path_factory)[mode]
    assert rows
    for step, got, want in rows:
        T.check_rows(got, want, dtype, f"{name} {dtype} {mode} step {step}")


def test_mixed_trace_has_portions_beside_decoded_tokens_and_four_live_requests():
    reqs = T.requests_for(256, LENGTHS["A"], seed=1)
    trace, peak = T.trace_mixed(reqs, seed=7)
    sizes = [[len(e["tokens"]) for e in s["entries"]] for s in trace.steps]
    assert any(len(s) == 4 for s in sizes)
    assert any(1 in s and max(s) > 1 for s in sizes)
    assert any(2 in s for s in sizes) or any(2 in [len(e["tokens"]) for e in st["entries"]]
                                              for st in T.trace_portions(reqs, 5).steps)
    assert peak < sum(T.rounded(len(t)) for t in reqs.values())
