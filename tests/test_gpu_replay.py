"""Replay through `bin/trace_run`: the same requests whole, with the last 32 tokens decoded one by one,
in portions of changing size, and mixed with other requests in a pool so small that pages are used
again; in float32 and in bfloat16; each compared with the plain implementation, and in float32 the four
ways of cutting with each other, bit for bit.  Every configuration is replayed with the page size that
goes with it (A: pages of 4)."""
import functools
import os

import pytest
import torch
from conftest import SHAPES

import plain_qwen3 as P
import trace_tools as T

pytestmark = pytest.mark.gpu

LENGTHS = {"A": [70, 45, 33, 100, 130, 64, 37, 90], "B": [1, 7, 17, 40, 129, 65, 96, 50], "C": [48, 80, 35, 66, 120],
           "D": [70, 45, 200, 33, 300, 131, 64], "R": [70, 45, 131, 64, 37], "S": [150, 33, 161, 18, 47, 129, 55]}
MODES = ("whole", "decode_tail", "portions", "mixed")
# "S": configuration D with the q and k head norms' weights scaled so that attention is peaked: one key read from a
# wrong page or place moves the logits by far more than the bfloat16 gate allows (with the random weights as drawn,
# attention is nearly uniform and a misplaced key hides below the gate).  Factor 3 in float32; in bfloat16 the rounding
# of q and k grows with the scores, so 1.5 (the reference's own rounding chain moves the logits by an NRMSE of 0.03 there).
SHARPENING = {"float32": 3.0, "bfloat16": 1.5}


def shape_of(name):
    return SHAPES["D" if name == "S" else name]


@functools.lru_cache(maxsize=None)
def plain_logits(folder: str, name: str):
    cfg, weights = P.PlainConfig.load(folder), P.load_plain_weights(folder)
    reqs = T.requests_for(cfg.vocab_size, LENGTHS[name], seed=100 + ord(name))
    return reqs, {r: P.logits_of_sequence(cfg, weights, tokens) for r, tokens in reqs.items()}


_results = {}
_sharp_folders = {}


def folder_of(request, model_folders, tmp_path_factory, name, dtype):
    if name == "R":
        return request.getfixturevalue("real_size_folder")
    if name == "S":
        if dtype not in _sharp_folders:
            _sharp_folders[dtype] = T.sharpen(model_folders["D"], str(tmp_path_factory.mktemp(f"sharp_{dtype}")), SHARPENING[dtype])
        return _sharp_folders[dtype]
    return model_folders[name]


def replay(folder: str, name: str, dtype: str, tmp_path_factory):
    """All four traces of one configuration and dtype through one trace_run process.  For every mode the steps
    with wanted rows: (step, logits, plain logits, [(request, position) of each row])."""
    key = (name, dtype)
    if key in _results:
        return _results[key]
    reqs, want = plain_logits(folder, name)
    raw, page = shape_of(name)
    vocab = raw["vocab_size"]
    mixed, peak = T.trace_mixed(reqs, seed=7)
    traces = {"whole": T.trace_whole(reqs), "decode_tail": T.trace_decode_tail(reqs),
              "portions": T.trace_portions(reqs, seed=5), "mixed": mixed}
    max_tokens = max(peak, max(T.rounded(len(t)) for t in reqs.values()))
    assert sum(T.rounded(len(t)) for t in reqs.values()) > max_tokens, "the pool must force pages to be used again"
    run = T.TraceRun(folder, dtype, str(tmp_path_factory.mktemp(f"out_{name}_{dtype}")), max_tokens,
                     extra=("--page-size", str(page)))
    out = {}
    first = 0
    for mode in MODES:
        trace = T.renumber(traces[mode], first, f"{mode}-")
        first += len(trace.steps)
        rows = []
        for step, places in zip(trace.steps, trace.rows):
            got = run.step(step, vocab)
            if places:
                rows.append((step["step"], got, torch.stack([want[r][p] for r, p in places]), places))
        out[mode] = rows
    assert run.close() == 0
    _results[key] = out
    return out


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "R", "S"])
def test_replay_matches_plain(request, model_folders, tmp_path_factory, name, dtype, mode):
    """"R": two layers of a real checkpoint's sizes, so that every cutting also runs at the sizes of production.
    "S": peaked attention, so that one wrong page shows in bfloat16 too."""
    folder = folder_of(request, model_folders, tmp_path_factory, name, dtype)
    rows = replay(folder, name, dtype, tmp_path_factory)[mode]
    assert rows
    for step, got, want, _ in rows:
        T.check_rows(got, want, dtype, f"{name} {dtype} {mode} step {step}")


@pytest.mark.parametrize("name", ["A", "B", "C", "D", "R", "S"])
def test_float32_logits_do_not_depend_on_the_cutting_bit_for_bit(request, model_folders, tmp_path_factory, name):
    """The reference's invariant (scripts/verify_model.py:158-170, `chunked_logits_exact`): the logits of a
    position are the same bits whether the request ran whole, token by token, in portions or beside other
    requests on reused pages.  It holds on the 32-bit path because every kernel's sum for a row runs in an order
    that depends on the row alone."""
    folder = folder_of(request, model_folders, tmp_path_factory, name, "float32")
    result = replay(folder, name, "float32", tmp_path_factory)
    whole = {}
    for _, got, _, places in result["whole"]:
        for row, place in zip(got, places):
            whole[place] = row
    compared = 0
    for mode in MODES[1:]:
        differing = []
        for step, got, _, places in result[mode]:
            for row, place in zip(got, places):
                if not torch.equal(row, whole[place]):
                    differing.append((step, place, (row - whole[place]).abs().max().item()))
                compared += 1
        assert not differing, f"{name} {mode}: {len(differing)} rows differ from the whole run, first {differing[:3]}"
    assert compared > 50


def test_mixed_trace_has_portions_beside_decoded_tokens_and_four_live_requests():
    reqs = T.requests_for(256, LENGTHS["A"], seed=1)
    trace, peak = T.trace_mixed(reqs, seed=7)
    sizes = [[len(e["tokens"]) for e in s["entries"]] for s in trace.steps]
    assert any(len(s) == 4 for s in sizes)
    assert any(1 in s and max(s) > 1 for s in sizes)
    assert any(2 in s for s in sizes) or any(2 in [len(e["tokens"]) for e in st["entries"]]
                                              for st in T.trace_portions(reqs, 5).steps)
    assert peak < sum(T.rounded(len(t)) for t in reqs.values())


def test_trace_run_takes_the_page_size_and_refuses_a_bad_one(model_folders, tmp_path):
    """Pages of 4 (configuration A's own): 64 tokens are 16 pages, and a trace that overruns them fails loudly."""
    folder = model_folders["A"]
    run = T.TraceRun(folder, "float32", str(tmp_path / "out"), 64, extra=("--page-size", "4"))
    cfg, weights = P.PlainConfig.load(folder), P.load_plain_weights(folder)
    tokens = list(range(3, 63))
    got = run.step({"step": 0, "entries": [{"id": "a", "tokens": tokens, "want": [0, 59]}], "end": []}, cfg.vocab_size)
    T.check_rows(got, P.logits_of_sequence(cfg, weights, tokens)[[0, 59]], "float32", "pages of 4")
    run.proc.stdin.write('{"step": 1, "entries": [{"id": "b", "tokens": [1, 2, 3, 4, 5, 6, 7, 8, 9], "want": []}], "end": []}\n')
    run.proc.stdin.flush()
    assert run.proc.stdout.readline() == ""            # 60 + 9 tokens need 18 pages of 4, the pool has 16
    assert run.close() == 1
    import subprocess
    import sys
    bad = subprocess.run([sys.executable, T.TRACE_RUN, "--model", folder, "--dtype", "float32", "--out", str(tmp_path / "o2"),
                          "--max-tokens", "64", "--page-size", "12"], input="", capture_output=True, text=True, timeout=300)
    assert bad.returncode == 1 and "power of two" in bad.stderr
