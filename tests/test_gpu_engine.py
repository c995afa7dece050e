"""The engine in process: cuttings with the tiny configurations' own page sizes, page reuse with
weights that make a wrong key show, long decoding, first tokens, generation through the entry
point and the command line."""
import json
import os
import subprocess
import sys

import pytest
import torch
from conftest import ROOT, TINY

import plain_qwen3 as P
import trace_tools as T
from mini_rsglang_b200 import RuntimeConfig, SamplingParams
from mini_rsglang_b200.engine import EngineHandle, GenerateRequest, ModelRunner, SequenceStep, Token, TokenIds, Finished

pytestmark = pytest.mark.gpu


def runner_for(folder, name, dtype, pages=64, max_seq_len=1024, running=4):
    limits = RuntimeConfig(max_seq_len=max_seq_len, page_size=TINY[name][1], max_running=running)
    return ModelRunner.load(folder, dtype=dtype, limits=limits, num_pages=pages)


def plain(folder, tokens):
    return P.logits_of_sequence(P.PlainConfig.load(folder), P.load_plain_weights(folder), tokens)


def feed(runner, request, tokens, cuts, want_all=True):
    """Feeds `tokens` of one request in portions of the given sizes; returns logits of every position."""
    out, pos = [], 0
    runner.cache.open(request)
    for n in cuts:
        runner.cache.extend(request, pos + n)
        out.append(runner.step([SequenceStep(request, tokens[pos:pos + n], pos, list(range(n)))]).double().cpu())
        pos += n
    assert pos == len(tokens)
    return torch.cat(out)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_first_tokens_of_a_sequence(model_folders, name, dtype):
    """Positions 0, 1, 2: one key, the first page, no rotation at position 0."""
    runner = runner_for(model_folders[name], name, dtype)
    tokens = [5, 9, 2]
    want = plain(model_folders[name], tokens)
    T.check_rows(feed(runner, 1, tokens, [3]), want, dtype, "first tokens whole")
    T.check_rows(feed(runner, 2, tokens, [1, 1, 1]), want, dtype, "first tokens one by one")
    one = feed(runner, 3, tokens[:1], [1])
    T.check_rows(one, want[:1], dtype, "a prompt of one token")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_page_edges_with_the_configurations_own_page_size(model_folders, name, dtype):
    """Cuts that end exactly at, one before and one after a page's edge."""
    page = TINY[name][1]
    runner = runner_for(model_folders[name], name, dtype)
    vocab = TINY[name][0]["vocab_size"]
    tokens = [(7 * i + 3) % vocab for i in range(4 * page + 3)]
    want = plain(model_folders[name], tokens)
    cuts = [page - 1, 1, 1, page, page + 1, page - 2]
    cuts.append(len(tokens) - sum(cuts))
    T.check_rows(feed(runner, 1, tokens, cuts), want, dtype, f"{name} page edges")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(model_folders, dtype):
    """A short prompt, then 300 tokens one by one: rounding must not build up, pages keep coming."""
    name = "B"
    runner = runner_for(model_folders[name], name, dtype)
    vocab = TINY[name][0]["vocab_size"]
    tokens = [(11 * i + 5) % vocab for i in range(310)]
    want = plain(model_folders[name], tokens)
    got = feed(runner, 1, tokens, [10] + [1] * 300)
    T.check_rows(got, want, dtype, "long decoding")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["B", "D"])
def test_recorded_decode_steps_equal_queued_ones(model_folders, name, dtype):
    """Three requests of different lengths decode together: the step is padded to four rows,
    recorded once and replayed.  Logits equal those of a runner that queues every kernel (bit
    for bit in float32) and the plain implementation's."""
    vocab = TINY[name][0]["vocab_size"]
    reqs = T.requests_for(vocab, [60, 23, 41], seed=9)
    want = {r: plain(model_folders[name], t) for r, t in reqs.items()}
    heads = {"r0": 30, "r1": 3, "r2": 17}
    results = []
    for record in (True, False):
        runner = runner_for(model_folders[name], name, dtype)
        assert runner.record_decode
        runner.record_decode = record
        for i, (r, tokens) in enumerate(reqs.items()):
            runner.cache.open(i + 1)
            runner.cache.extend(i + 1, heads[r])
            runner.step([SequenceStep(i + 1, tokens[:heads[r]], 0, [])])
        rows = []
        for k in range(20):
            batch = []
            for i, (r, tokens) in enumerate(reqs.items()):
                runner.cache.extend(i + 1, heads[r] + k + 1)
                batch.append(SequenceStep(i + 1, [tokens[heads[r] + k]], heads[r] + k, [0]))
            got = runner.step(batch).double().cpu()
            T.check_rows(got, torch.stack([want[r][heads[r] + k] for r in reqs]), dtype, f"decode step {k} (recorded={record})")
            rows.append(got)
        if record:
            assert len(runner._records) == 1 and next(iter(runner._records))[0] == 4
        results.append(torch.stack(rows))
    if dtype == "float32":
        assert torch.equal(results[0], results[1])


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


@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("B", "float32"), ("D", "float32"), ("D", "bfloat16")])
def test_reused_pages_with_peaked_attention(model_folders, tmp_path, name, dtype):
    """Requests come and go in a pool that holds two of them, so every page is written by several
    requests in turn and block tables are out of order; with peaked attention a stale or
    misplaced key would change the logits at once.  Configuration D runs it through the serving
    kernels as well (bfloat16, heads of 128)."""
    # factor 3: scores grow ninefold; float32 rounding of a score of that size stays below the gate.  In
    # bfloat16 the rounding of q and k grows with the scores as well (the reference's own rounding chain,
    # restated by the plain implementation, moves the logits of this model by an NRMSE of 0.16 at factor 3
    # and 0.03 at factor 1.5), so the bfloat16 run sharpens by 1.5 only.
    folder = sharpen(model_folders[name], str(tmp_path / "sharp"), 3.0 if dtype == "float32" else 1.5)
    cfg, weights = P.PlainConfig.load(folder), P.load_plain_weights(folder)
    page = TINY[name][1]
    lengths = [50, 33, 61, 18, 47, 29, 55] if name != "D" else [150, 33, 161, 18, 47, 129, 55]
    reqs = T.requests_for(cfg.vocab_size, lengths, seed=3)
    pool_pages = 2 * (-(-max(lengths) // page)) + 1
    limits = RuntimeConfig(max_seq_len=512, page_size=page, max_running=4)
    runner = ModelRunner.load(folder, dtype=dtype, limits=limits, num_pages=pool_pages)
    cache = runner.cache
    queue, live, fed = list(reqs), {}, {}
    ids = {r: i + 1 for i, r in enumerate(reqs)}
    seen_tables = []
    import random
    rng = random.Random(4)
    while queue or live:
        while queue and len(live) < 3:
            need = -(-len(reqs[queue[0]]) // page)
            held = sum(-(-len(reqs[r]) // page) for r in live)
            if held + need > pool_pages:
                break
            live[queue.pop(0)] = 0
            cache.open(ids[list(live)[-1]])
        batch, places = [], []
        for r in list(live):
            p, tokens = live[r], reqs[r]
            n = min(rng.choice([1, 2, 3, 7, 12] if name != "D" else [1, 1, 2, 7, 40, 70]), len(tokens) - p)
            cache.extend(ids[r], p + n)
            batch.append(SequenceStep(ids[r], tokens[p:p + n], p, [n - 1]))
            places.append((r, p + n - 1))
            live[r] = p + n
        got = runner.step(batch).double().cpu()
        want = torch.stack([P.logits_of_sequence(cfg, weights, reqs[r][:p + 1])[-1] for r, p in places])
        T.check_rows(got, want, dtype, f"{name} reuse")
        for r in list(live):
            if live[r] == len(reqs[r]):
                seen_tables.append(list(cache.table(ids[r])))
                cache.close(ids[r])
                del live[r]
        cache.check_integrity()
    assert any(t != sorted(t) or t[0] != 0 for t in seen_tables[1:]), "block tables never left the natural order"
    used = [p for t in seen_tables for p in t]
    assert len(used) > pool_pages                       # pages were used again


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "D"])
def test_greedy_generation_through_the_entry_point(model_folders, name, dtype):
    folder = model_folders[name]
    cfg, weights = P.PlainConfig.load(folder), P.load_plain_weights(folder)
    limits = RuntimeConfig(max_seq_len=256, page_size=TINY[name][1], prefill_budget=8, max_running=3)
    engine = EngineHandle.load(folder, 0, config=limits, dtype=dtype, num_pages=40)
    prompts = [[3, 1, 4, 1, 5], [9, 2, 6, 5, 3, 5, 8, 9, 7], [2, 7, 1, 8, 2, 8, 1, 8, 2, 8, 4, 5, 9], [6]]
    steps = 8
    results = engine.generate_many(prompts, SamplingParams(max_tokens=steps, ignore_eos=True))
    for prompt, result in zip(prompts, results):
        assert result.finish_reason == "length" and result.prompt_tokens == len(prompt)
        # follow the engine's tokens; at every step they must be the plain arg-max unless the two
        # best plain logits are closer than the path's rounding
        tokens = list(prompt)
        for token in result.token_ids:
            logits = P.logits_of_sequence(cfg, weights, tokens)[-1]
            best = P.greedy(logits)
            if token != best:
                gap = (logits[best] - logits[token]).item()
                allowed = 2e-5 if dtype == "float32" else 0.02 * logits.abs().max().item()
                assert gap <= allowed, f"token {token} instead of {best}, gap {gap}"
            tokens.append(token)
    assert engine.runner.cache.free_pages() == 40
    metrics = engine.metrics()
    assert metrics["completed"] == 4 and metrics["generated_tokens"] == 4 * steps and metrics["mixed_batches"] > 0
    engine.shutdown()


def test_streams_events_stop_reason_and_seeded_sampling(model_folders):
    folder = model_folders["B"]
    limits = RuntimeConfig(max_seq_len=128, page_size=16, prefill_budget=8, max_running=4)
    engine = EngineHandle.load(folder, 0, config=limits, dtype="bfloat16", num_pages=32)
    # temperature 0.7, seeded: the same seed gives the same tokens whatever else runs beside it
    params = SamplingParams(temperature=0.7, seed=1234, max_tokens=6, ignore_eos=True)
    alone = engine.generate_many([[5, 6, 7, 8]], params)[0].token_ids
    beside = engine.generate_many([[1, 2, 3], [5, 6, 7, 8], [9] * 20],
                                  [SamplingParams(max_tokens=9, ignore_eos=True), params,
                                   SamplingParams(temperature=1.0, seed=5, max_tokens=3, ignore_eos=True)])
    assert beside[1].token_ids == alone
    other_seed = engine.generate_many([[5, 6, 7, 8]], SamplingParams(temperature=0.7, seed=99, max_tokens=6, ignore_eos=True))
    assert other_seed[0].token_ids != alone
    # events of one stream, and an end-of-sequence token stops it
    stream = engine.generate(GenerateRequest(TokenIds([5, 6, 7, 8]), SamplingParams(max_tokens=4, ignore_eos=True)))
    events = list(stream)
    assert [type(e) for e in events] == [Token] * 4 + [Finished] and events[-1].reason == "length"
    first = events[0].token_id
    engine.scheduler = type(engine.scheduler)(engine.runner.cache, limits, [first], 384)
    stopped = engine.generate_many([[5, 6, 7, 8]], SamplingParams(max_tokens=4))[0]
    assert stopped.finish_reason == "stop" and stopped.token_ids == [first]
    engine.shutdown()
    from mini_rsglang_b200 import EngineStopped
    with pytest.raises(EngineStopped):
        engine.generate(GenerateRequest(TokenIds([1]), SamplingParams()))


def test_refusals_of_the_entry_point_and_the_step_function(model_folders):
    from mini_rsglang_b200 import CapacityError, InvalidRequest
    folder = model_folders["A"]
    limits = RuntimeConfig(max_seq_len=64, page_size=4, prefill_budget=8, max_running=2, max_waiting=2)
    engine = EngineHandle.load(folder, 0, config=limits, dtype="float32", num_pages=8)
    with pytest.raises(InvalidRequest):
        engine.generate(GenerateRequest(TokenIds([]), SamplingParams()))
    with pytest.raises(InvalidRequest):
        engine.generate(GenerateRequest(TokenIds([256]), SamplingParams(max_tokens=2)))
    with pytest.raises(InvalidRequest, match="context limit"):
        engine.generate(GenerateRequest(TokenIds([1] * 60), SamplingParams(max_tokens=8)))
    with pytest.raises(CapacityError):
        engine.generate(GenerateRequest(TokenIds([1] * 30), SamplingParams(max_tokens=8)))   # 10 pages > 8
    runner = engine.runner
    runner.cache.open(77)
    runner.cache.extend(77, 4)
    with pytest.raises(InvalidRequest, match="appears twice"):
        runner.step([SequenceStep(77, [1, 2], 0), SequenceStep(77, [3], 2)])
    with pytest.raises(InvalidRequest, match="coverage"):
        runner.step([SequenceStep(77, [1] * 6, 0)])
    with pytest.raises(InvalidRequest, match="out of range"):
        runner.step([SequenceStep(77, [999], 0)])
    with pytest.raises(InvalidRequest):
        runner.step([])
    runner.cache.close(77)
    with pytest.raises(InvalidRequest, match="max_position_embeddings"):
        EngineHandle.load(folder, 0, config=RuntimeConfig(max_seq_len=4096), dtype="float32", num_pages=8)


def test_command_line_generates_what_the_entry_point_generates(model_folders, tmp_path):
    folder = model_folders["A"]
    cmd = [sys.executable, os.path.join(ROOT, "bin", "mini-rsglang"), "--model", folder, "--dtype", "float32",
           "--page-size", "4", "--max-seq-len", "128", "--num-pages", "32", "generate", "--token-ids", "3,1,4,1,5",
           "--max-tokens", "5", "--ignore-eos", "--json"]
    proc = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    assert proc.returncode == 0, proc.stderr
    events = [json.loads(line) for line in proc.stdout.splitlines() if line.startswith("{")]
    tokens = [e["Token"]["token_id"] for e in events if "Token" in e]
    done = events[-1]["Finished"]
    assert done["reason"] == "length" and done["prompt_tokens"] == 5 and done["completion_tokens"] == 5
    cfg, weights = P.PlainConfig.load(folder), P.load_plain_weights(folder)
    assert tokens == P.generate_greedy(cfg, weights, [3, 1, 4, 1, 5], 5)
    bad = subprocess.run(cmd[:-6] + ["--token-ids", "3,x", "--max-tokens", "5"], capture_output=True, text=True, timeout=300)
    assert bad.returncode != 0 and "comma-separated integers" in bad.stderr


def test_command_line_load_test_reports_fixed_lengths(model_folders, tmp_path):
    """`bench` as the reference has it: a closed loop of requests of fixed lengths; every request ends at
    its length, the counts add up, and the report goes to standard output and to --output."""
    folder = model_folders["B"]
    out = tmp_path / "report.json"
    cmd = [sys.executable, os.path.join(ROOT, "bin", "mini-rsglang"), "--model", folder, "--page-size", "16",
           "--max-seq-len", "128", "--num-pages", "40", "--max-running", "4", "--prefill-budget", "32", "bench",
           "--input-tokens", "37", "--output-tokens", "6", "--requests", "7", "--concurrency", "3", "--output", str(out)]
    proc = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    assert proc.returncode == 0, proc.stderr
    report = json.loads(out.read_text())
    assert json.loads(proc.stdout[proc.stdout.index("{"):]) == report
    run = report["runs"][0]
    assert (run["requests"], run["concurrency"], run["input_tokens"], run["output_tokens"]) == (7, 3, 37, 6)
    assert len(run["raw_ttft_s"]) == 7 and len(run["raw_latency_s"]) == 7 and len(run["raw_itl_s"]) == 7 * 5
    assert run["output_tokens_per_s"] > 0 and run["ttft_ms"]["p50"] <= run["latency_ms"]["p50"]
    assert run["metrics"]["running"] == 0 and run["metrics"]["waiting"] == 0
    refused = subprocess.run(cmd[:-2] + ["--concurrency", "9"], capture_output=True, text=True, timeout=300)
    assert refused.returncode != 0 and "concurrency must be <= max_running" in refused.stderr
    hot = subprocess.run(cmd[:-2] + ["--cache-mode", "hot"], capture_output=True, text=True, timeout=300)
    assert hot.returncode != 0 and "no prefix cache" in hot.stderr


def test_portions_of_a_long_prompt_share_their_keys(model_folders, monkeypatch):
    """A prompt of 1,500 tokens in portions of 256 and 100 with heads of 128: from the second thousand on a portion makes
    few CTAs with many key blocks each, and the plan cuts its entries into shares of the keys, which a second kernel
    merges.  The logits of every portion's tokens equal the plain implementation's; the early portions, with few
    blocks, take entries of one tile."""
    from mini_rsglang_b200 import kernels

    folder = model_folders["D"]
    runner = runner_for(folder, "D", "bfloat16", pages=120, max_seq_len=2048)
    tokens = T.requests_for(TINY["D"][0]["vocab_size"], [1500], seed=31)["r0"]
    want = plain(folder, tokens)
    calls = []
    real = kernels.attention_prefill_tc
    monkeypatch.setattr(kernels, "attention_prefill_tc", lambda *a, **k: (calls.append((a[5].cpu().tolist(), k.get("shares"))), real(*a, **k))[1])
    got = feed(runner, 1, tokens, [256, 256, 256, 256, 256, 100, 120])
    T.check_rows(got, want, "bfloat16", "portions whose entries share their keys")
    shared = [tiles for tiles, shares in calls if shares]
    assert shared and all((t[3] >> 8) >= 2 for tiles in shared for t in tiles if t[3])
    assert any(not shares and all(t[2] <= 64 for t in tiles) for tiles, shares in calls)      # one tile: 128 rows / 2 heads of a group


def test_gate_up_product_for_many_rows_carries_the_activation(model_folders, monkeypatch):
    """With many rows the gate/up product runs on the tcgen05 kernel for many rows, with the activation in its epilogue
    (from 2,048 rows on; here from 64 on, so that a tiny model takes the path): the same logits as the plain
    implementation, whole and in portions."""
    from mini_rsglang_b200 import kernels

    monkeypatch.setattr(kernels, "GEMM_GATED_ROWS_MIN", 64)
    used = []
    real = kernels.gemm_gated_rows
    monkeypatch.setattr(kernels, "gemm_gated_rows", lambda *a, **k: (used.append("gemm_gated_rows"), real(*a, **k))[1])
    folder = model_folders["D"]
    runner = runner_for(folder, "D", "bfloat16", pages=64, max_seq_len=1024)
    tokens = T.requests_for(TINY["D"][0]["vocab_size"], [333], seed=41)["r0"]
    want = plain(folder, tokens)
    T.check_rows(feed(runner, 1, tokens, [333]), want, "bfloat16", "many rows, whole")
    T.check_rows(feed(runner, 2, tokens, [200, 70, 63]), want, "bfloat16", "many rows, portions (the last one below the limit)")
    assert len(used) == 2 * 3      # two layers, three steps at or above 64 rows
