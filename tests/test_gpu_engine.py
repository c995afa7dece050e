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
            decode_records = [key for key in runner._records if len(key) == 2]
            assert len(decode_records) == 1 and decode_records[0][0] == 4
        results.append(torch.stack(rows))
    if dtype == "float32":
        assert torch.equal(results[0], results[1])


def mixed_schedule(lengths, decoded, budget, caps):
    """Steps of a small continuous batch, as the scheduler would cut them: every request whose prompt is in
    decodes one token a step, the others bring portions of their prompts (at most `caps[k]` tokens in step k)
    under a budget of tokens a step.  Entries: (request index, first position, tokens, wanted place or None)."""
    done = [0] * len(lengths)
    steps, k = [], 0
    while any(d < n + decoded for d, n in zip(done, lengths)):
        left, step = budget, []
        for i, n in enumerate(lengths):
            if n <= done[i] < n + decoded and left > 0:
                step.append((i, done[i], 1, 0))
                left -= 1
        for i, n in enumerate(lengths):
            if done[i] < n and left > 0:
                take = min(n - done[i], left, caps[k % len(caps)])
                step.append((i, done[i], take, take - 1 if done[i] + take == n else None))
                left -= take
        for i, _, take, _ in step:
            done[i] += take
        steps.append(step)
        k += 1
    return steps


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "D"])
def test_recorded_steps_with_prompt_portions_equal_queued_ones(model_folders, name, dtype):
    """Steps that hold portions of prompts beside decoded tokens are padded to fixed shapes, recorded once per
    shape and replayed.  Every wanted row equals the plain implementation's, and in float32 the rows of a runner
    that queues every kernel bit for bit; shapes come back, so recordings are replayed with other contents, in
    other pages and with other tile lists."""
    vocab = TINY[name][0]["vocab_size"]
    lengths = [90, 70, 50, 33]
    reqs = list(T.requests_for(vocab, [n + 12 for n in lengths], seed=31).values())
    want = [plain(model_folders[name], tokens) for tokens in reqs]
    steps = mixed_schedule(lengths, 12, 40, [13, 24, 17, 20, 9])
    results = []
    for record in (True, False, "few"):
        runner = runner_for(model_folders[name], name, dtype, pages=128)
        assert runner.record_mixed
        runner.record_mixed = bool(record)
        if record == "few":                  # room for two recordings: every other shape is queued kernel by kernel
            runner.max_records = 2
        for i in range(len(reqs)):
            runner.cache.open(i + 1)
        rows = []
        for k, step in enumerate(steps):
            batch = []
            for i, first, take, place in step:
                runner.cache.extend(i + 1, first + take)
                batch.append(SequenceStep(i + 1, reqs[i][first:first + take], first, [] if place is None else [place]))
            got = runner.step(batch)
            wanted = [(i, first + place) for i, first, _, place in step if place is not None]
            assert (got is None) == (not wanted)
            if wanted:
                got = got.double().cpu()
                T.check_rows(got, torch.stack([want[i][p] for i, p in wanted]), dtype, f"step {k} (recorded={record})")
                rows.append(got)
        if record == "few":
            assert 1 <= len([key for key in runner._records if len(key) == 5]) <= 2 and runner.recorded_steps < len(steps)
        elif record:
            fixed = [key for key in runner._records if len(key) == 5]
            mixed_steps = sum(1 for step in steps if any(take > 1 for _, _, take, _ in step))
            assert len(fixed) >= 3 and mixed_steps > len(fixed)               # recordings were replayed
            assert runner.recorded_steps == len(steps)
        results.append(torch.cat(rows))
    if dtype == "float32":
        assert torch.equal(results[0], results[1]) and torch.equal(results[0], results[2])


def test_the_two_attention_kernels_of_a_mixed_step_side_by_side_give_what_they_give_one_after_the_other(model_folders, monkeypatch):
    """Decoded tokens beside prompt portions: the attention for few rows runs on a second stream beside the one for
    prompt portions.  The logits are, bit for bit, those of the two kernels run one after the other, queued and
    recorded."""
    from mini_rsglang_b200.parts import attention
    name, dtype = "D", "bfloat16"
    vocab = TINY[name][0]["vocab_size"]
    lengths = [150, 90, 40]
    reqs = list(T.requests_for(vocab, [n + 6 for n in lengths], seed=53).values())
    steps = mixed_schedule(lengths, 6, 64, [40, 33, 50])
    results = []
    for side_by_side, record in ((True, True), (False, True), (True, False), (False, False)):
        monkeypatch.setattr(attention, "SIDE_BY_SIDE", side_by_side)
        runner = runner_for(model_folders[name], name, dtype, pages=128)
        runner.record_mixed = runner.record_decode = record
        for i in range(len(reqs)):
            runner.cache.open(i + 1)
        rows = []
        for step in steps:
            batch = []
            for i, first, take, place in step:
                runner.cache.extend(i + 1, first + take)
                batch.append(SequenceStep(i + 1, reqs[i][first:first + take], first, [] if place is None else [place]))
            got = runner.step(batch)
            if got is not None:
                rows.append(got.cpu())
        results.append(torch.cat(rows))
    assert any(len(step) > 1 and any(take > 1 for _, _, take, _ in step) and any(take == 1 for _, _, take, _ in step) for step in steps)
    assert torch.equal(results[0], results[1]) and torch.equal(results[2], results[3])


def test_generation_through_recorded_steps_with_portions(model_folders):
    """The entry point with a small token budget: its mixed steps are recorded (every shape at its first use)
    and the tokens are the ones that a runner without recordings generates."""
    folder = model_folders["D"]
    prompts = [[(3 * i + k) % 500 + 4 for i in range(n)] for k, n in enumerate([70, 45, 100, 12, 64, 33])]
    out = []
    for record in (True, False):
        limits = RuntimeConfig(max_seq_len=256, page_size=16, prefill_budget=48, max_running=4, record_mixed_steps=record)
        engine = EngineHandle.load(folder, 0, config=limits, dtype="float32", num_pages=80)
        results = engine.generate_many(prompts, SamplingParams(max_tokens=10, ignore_eos=True))
        out.append([r.token_ids for r in results])
        if record:
            assert any(len(key) == 5 for key in engine.runner._records)
        assert engine.runner.cache.free_pages() == 80
        engine.shutdown()
    assert out[0] == out[1]


sharpen = T.sharpen


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


@pytest.mark.parametrize("name", ["B", "D"])
def test_float32_tokens_do_not_depend_on_pages_budget_or_concurrency(model_folders, name):
    """The same prompts through engines with other page sizes, token budgets, numbers of requests in flight, with and
    without shared prefixes, recordings and overlapped steps: in float32 every engine generates the same tokens,
    since a row's arithmetic does not depend on how the tokens were cut or where in the cache they lie."""
    import random
    folder = model_folders[name]
    vocab = TINY[name][0]["vocab_size"]
    rng = random.Random(8)
    family = [rng.randrange(vocab) for _ in range(200)]
    prompts = [[rng.randrange(vocab) for _ in range(n)] for n in (1, 2, 17, 100, 260)] + [family[:150], family[:190] + [3, 4], family[:64]]
    outputs = []
    settings = [dict(page_size=16, prefill_budget=512, max_running=32), dict(page_size=8, prefill_budget=9, max_running=2),
                dict(page_size=4, prefill_budget=64, max_running=3, prefix_cache=True),
                dict(page_size=32, prefill_budget=2048, max_running=8, record_mixed_steps=False),
                dict(page_size=64, prefill_budget=100, max_running=5, overlap_steps=False, prefix_cache=True),
                dict(page_size=128, prefill_budget=300, max_running=4)]
    for setting in settings:
        limits = RuntimeConfig(max_seq_len=512, max_waiting=64, **setting)
        engine = EngineHandle.load(folder, 0, config=limits, dtype="float32", num_pages=40 * 512 // setting["page_size"])
        results = engine.generate_many(prompts, SamplingParams(max_tokens=12, ignore_eos=True))
        outputs.append([r.token_ids for r in results])
        engine.shutdown()
    for setting, output in zip(settings[1:], outputs[1:]):
        assert output == outputs[0], f"other tokens with {setting}"


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
    # --random-weights SEED: only config.json is read; the same seed gives the same tokens
    only_config = tmp_path / "only_config"
    only_config.mkdir()
    (only_config / "config.json").write_text(open(os.path.join(folder, "config.json")).read())
    runs = []
    for seed in ("5", "5"):
        random_cmd = [cmd[0], cmd[1], "--model", str(only_config), "--random-weights", seed] + cmd[4:-1]
        proc = subprocess.run(random_cmd, capture_output=True, text=True, timeout=300)
        assert proc.returncode == 0, proc.stderr
        runs.append(proc.stdout.strip().splitlines()[0])
    assert runs[0] == runs[1] and len(runs[0].split(",")) == 5


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
    assert hot.returncode == 0, hot.stderr
    run = json.loads(hot.stdout[hot.stdout.index("{"):])["runs"][0]
    # every request brings the prompt that is in the cache: 32 of its 37 tokens lie in full pages and are not computed
    assert run["cache_mode"] == "warm_prefix" and run["cached_tokens"] == 7 * 32
    assert len(run["raw_latency_s"]) == 7 and run["metrics"]["cached_pages"] >= 2


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_requests_that_share_their_first_tokens_read_them_from_the_cache(model_folders, dtype):
    """Prefix sharing through the entry point: prompts with common first pages, one after the other and side by
    side.  What a request reads from an earlier request's pages gives the tokens that computing it again gives
    (equal in float32, where the cutting changes no bit), the counts of cached tokens are the full pages before
    the last prompt token, and when the idle cache is cleared every page is free again."""
    name = "D"
    folder = model_folders[name]
    cfg, weights = P.PlainConfig.load(folder), P.load_plain_weights(folder)
    vocab = TINY[name][0]["vocab_size"]
    common = [(5 * i + 3) % vocab for i in range(50)]
    prompts = [common + [7, 8, 9], common[:40] + [1, 2], common + [7, 8, 9], [9] * 20, common[:17], common + [7, 8, 9, 10]]
    out = {}
    for share in (True, False):
        limits = RuntimeConfig(max_seq_len=256, page_size=16, prefill_budget=24, max_running=2, prefix_cache=share)
        engine = EngineHandle.load(folder, 0, config=limits, dtype=dtype, num_pages=40)
        first = engine.generate_many(prompts[:1], SamplingParams(max_tokens=5, ignore_eos=True))
        rest = engine.generate_many(prompts[1:], SamplingParams(max_tokens=5, ignore_eos=True))
        results = first + rest
        out[share] = [r.token_ids for r in results]
        if share:
            # full pages of 16 before the last prompt token that an earlier request had published
            assert [r.cached_tokens for r in results] == [0, 32, 48, 0, 16, 48]
            metrics = engine.metrics()
            assert metrics["cached_tokens"] == 144 and metrics["cached_pages"] > 0
            assert engine.runner.cache.free_pages() < 40
            engine.runner.cache.check_integrity()
            engine.clear_cache()
        else:
            assert all(r.cached_tokens == 0 for r in results)
        assert engine.runner.cache.free_pages() == 40
        engine.runner.cache.check_integrity()
        engine.shutdown()
    if dtype == "float32":
        assert out[True] == out[False]
    for prompt, generated in zip(prompts, out[True]):       # and the shared run's choices are the plain implementation's
        tokens = list(prompt)
        for token in generated:
            logits = P.logits_of_sequence(cfg, weights, tokens)[-1]
            best = P.greedy(logits)
            allowed = 2e-5 if dtype == "float32" else 0.02 * logits.abs().max().item()
            assert token == best or (logits[best] - logits[token]).item() <= allowed
            tokens.append(token)


@pytest.mark.parametrize("seed", [11, 12, 13])
def test_random_traffic_gives_the_same_tokens_with_and_without_recordings_and_sharing(model_folders, seed):
    """Random prompts from a few families of common first tokens, random lengths and output lengths, a small token
    budget and a page pool that holds only some of them at a time: in float32 an engine that records its steps and
    shares prefixes generates, token for token, what one that queues every kernel and shares nothing generates,
    whether or not steps are queued before the tokens of the step before them are known (stop tokens among them:
    half of the requests end on one); nothing leaks, and the manager's books balance after every wave."""
    import random
    name = "B"
    folder = model_folders[name]
    vocab = TINY[name][0]["vocab_size"]
    rng = random.Random(seed)
    families = [[rng.randrange(3, vocab) for _ in range(70)] for _ in range(3)]
    waves = []
    for _ in range(3):
        prompts, params = [], []
        for _ in range(rng.randrange(4, 9)):
            family = rng.choice(families)
            prompts.append(family[:rng.randrange(1, 70)] + [rng.randrange(3, vocab) for _ in range(rng.randrange(0, 9))])
            params.append(SamplingParams(max_tokens=rng.randrange(1, 12), ignore_eos=rng.random() < 0.5,
                                         temperature=rng.choice([0.0, 0.0, 0.8]), seed=rng.randrange(1 << 30)))
        waves.append((prompts, params))
    out = []
    for fancy, overlap in ((True, True), (False, False), (True, False), (False, True)):
        limits = RuntimeConfig(max_seq_len=128, page_size=16, prefill_budget=32, max_running=4,
                               prefix_cache=fancy, record_mixed_steps=fancy, overlap_steps=overlap)
        engine = EngineHandle.load(folder, 0, config=limits, dtype="float32", num_pages=24)
        engine.runner.record_decode = fancy
        tokens = []
        for prompts, params in waves:
            results = engine.generate_many(prompts, params)
            tokens.append([(r.token_ids, r.finish_reason) for r in results])
            engine.runner.cache.check_integrity()
        if fancy:
            assert engine.metrics()["cached_tokens"] > 0 and any(len(key) == 5 for key in engine.runner._records)
            engine.clear_cache()
        assert engine.runner.cache.free_pages() == 24
        engine.shutdown()
        out.append(tokens)
    assert out[0] == out[1] == out[2] == out[3]


def test_prefix_sharing_is_refused_for_a_model_that_cannot_share(model_folders):
    """A window of keys or a state of its own per request cannot be shared: asking for it fails at load."""
    from mini_rsglang_b200 import InvalidRequest
    import dataclasses
    from mini_rsglang_b200.models.registry import load_config, model_spec_for
    from mini_rsglang_b200.parts.base import PartSpec
    folder = model_folders["A"]
    config = load_config(folder)
    spec = model_spec_for(config)
    mixer = spec.layers[0].parts["mixer"]
    windowed = PartSpec(mixer.kind, {**mixer.params, "window": 8})
    spec.layers[0] = dataclasses.replace(spec.layers[0], parts={**spec.layers[0].parts, "mixer": windowed})
    limits = RuntimeConfig(max_seq_len=64, page_size=4, max_running=2, prefix_cache=True)
    from mini_rsglang_b200.parts.base import Runtime
    from mini_rsglang_b200.weights import load_weights
    runtime = Runtime(torch.device("cuda:0"), torch.float32, 4)
    tensors = load_weights(folder, spec.weight_specs(), runtime.dtype, runtime.device, spec.ignorable_weights)
    with pytest.raises(InvalidRequest, match="prefix sharing"):
        ModelRunner(config, tensors, runtime, limits, num_pages=16, spec=spec)


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


def test_the_gate_up_product_for_many_rows_is_chosen_by_a_measurement_kept_per_shape(monkeypatch):
    """From the least number of rows on, the tcgen05 gate/up product and the library's product with `silu_mul`
    are timed once for a shape and the faster one is kept; below it, and where the kernel cannot run, the library."""
    from mini_rsglang_b200 import kernels

    monkeypatch.setattr(kernels, "GEMM_GATED_ROWS_MIN", 256)
    monkeypatch.setattr(kernels, "GEMM_GATED_MEASURE", True)
    weight = (torch.randn(512, 256, device="cuda:0") / 16).to(torch.bfloat16)
    x = torch.randn(300, 256, device="cuda:0").to(torch.bfloat16)
    kernels._gated_rows_choice.clear()
    first = kernels.gemm_gated_rows_wins(x, weight)
    assert isinstance(first, bool) and len(kernels._gated_rows_choice) == 1
    assert kernels.gemm_gated_rows_wins(x, weight) is first and len(kernels._gated_rows_choice) == 1      # kept
    assert kernels.gemm_gated_rows_wins(x[:100], weight) is False                                            # too few rows
    assert kernels.gemm_gated_rows_wins(x, weight[:200]) is False                                            # no whole blocks
    kernels.check_device_errors()


def test_recorded_portions_of_long_prompts_share_their_keys_and_reuse_their_recording(model_folders):
    """Portions of 256 tokens of two long prompts, one wanted place at most a step: the steps are recorded with fixed
    shapes, entries that share their keys among them (the merge kernel is part of those recordings), and the second
    prompt replays what the first recorded, with other tile lists in other pages.  The wanted rows equal the plain
    implementation's, decoded tokens beside the last portions included."""
    folder = model_folders["D"]
    runner = runner_for(folder, "D", "bfloat16", pages=240, max_seq_len=2048)
    reqs = T.requests_for(TINY["D"][0]["vocab_size"], [1540, 1541], seed=47)
    for i, tokens in enumerate(reqs.values()):
        want = plain(folder, tokens)
        runner.cache.open(i + 1)
        records = len(runner._records)
        at = 0
        for n in [256] * 6:
            runner.cache.extend(i + 1, at + n)
            last = at + n == 1536
            got = runner.step([SequenceStep(i + 1, tokens[at:at + n], at, [n - 1] if last else [])])
            at += n
            assert (got is None) == (not last)
        T.check_rows(got.double().cpu(), want[1535:1536], "bfloat16", f"request {i}: the last portion's last row")
        for p in range(1536, len(tokens)):
            runner.cache.extend(i + 1, p + 1)
            got = runner.step([SequenceStep(i + 1, [tokens[p]], p, [0])])
            T.check_rows(got.double().cpu(), want[p:p + 1], "bfloat16", f"request {i}: decoded token at {p}")
        if i == 1:
            assert len(runner._records) == records              # nothing new was recorded for the second prompt
    fixed = [key for key in runner._records if len(key) == 5]
    assert any(signature[0][2] for key in fixed for signature in key[4] if signature[0]), fixed      # entries that share keys


def test_gate_up_product_for_many_rows_carries_the_activation(model_folders, monkeypatch):
    """With many rows the gate/up product runs on the tcgen05 kernel for many rows, with the activation in its epilogue
    (from 2,048 rows on; here from 64 on, so that a tiny model takes the path): the same logits as the plain
    implementation, whole and in portions."""
    from mini_rsglang_b200 import kernels

    monkeypatch.setattr(kernels, "GEMM_GATED_ROWS_MIN", 64)
    monkeypatch.setattr(kernels, "GEMM_GATED_MEASURE", False)      # the kernel, whatever the library would take here
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


def test_a_failed_step_ends_every_request_and_gives_every_page_back(model_folders):
    """The step function fails in the middle of a mixed run (the failure is made on the host: `forward` raises):
    every stream gets an `Error`, every page and promise goes back, the counters say so, and the engine takes
    no more requests (reference: crates/runtime/src/scheduler.rs:332-359 and its test at 614-635)."""
    from mini_rsglang_b200 import BackendError, EngineStopped
    from mini_rsglang_b200.engine import Error
    folder = model_folders["A"]
    limits = RuntimeConfig(max_seq_len=128, page_size=4, prefill_budget=8, max_running=2, max_waiting=8)
    engine = EngineHandle.load(folder, 0, config=limits, dtype="float32", num_pages=40)
    params = SamplingParams(max_tokens=12, ignore_eos=True)
    streams = [engine.generate(GenerateRequest(TokenIds(p), params)) for p in ([3, 1, 4, 1, 5, 9, 2, 6, 5, 3, 5], [2, 7, 1], [8] * 20)]
    for _ in range(4):
        assert engine.run_step()
    assert engine.scheduler.running() == 2 and engine.scheduler.waiting() == 1      # two run, the third waits
    assert engine.runner.cache.free_pages() < 40

    def broken(batch, observe=None, carried=None):
        raise BackendError("injected: the device fell over")

    engine.runner.forward = broken
    with pytest.raises(BackendError, match="injected"):
        engine.run_step()
    for stream in streams:
        events = list(stream.events)
        assert any(isinstance(e, Error) and "injected" in e.message for e in events)
        assert isinstance(events[-1], Finished) and events[-1].reason == "error"
    metrics = engine.metrics()
    assert metrics["failed"] == 3 and metrics["healthy"] is False
    assert metrics["free_pages"] == metrics["total_pages"] == 40 and metrics["running"] == 0 and metrics["waiting"] == 0
    assert engine.runner.cache.reserved_pages() == 0 and engine.runner.cache.open_requests() == 0
    engine.runner.cache.check_integrity()
    with pytest.raises(EngineStopped):
        engine.generate(GenerateRequest(TokenIds([1]), SamplingParams()))
    with pytest.raises(EngineStopped):
        engine.run_step()


def test_a_wait_that_runs_out_fails_the_step_and_leaves_the_device_usable(model_folders):
    """A kernel's bounded wait runs out (a one-warp kernel waits 65,536 clocks on a barrier at which nobody arrives,
    then returns by itself): the error word is raised, the next check fails the step loudly, the word is clear
    afterwards and the following steps are right.  Through the entry point the same word ends every request."""
    from mini_rsglang_b200 import BackendError, kernels
    from mini_rsglang_b200.engine import Error
    folder = model_folders["D"]
    runner = runner_for(folder, "D", "bfloat16")
    tokens = T.requests_for(TINY["D"][0]["vocab_size"], [40], seed=5)["r0"]
    want = plain(folder, tokens)
    runner.cache.open(1)
    runner.cache.extend(1, 30)
    T.check_rows(runner.step([SequenceStep(1, tokens[:30], 0, [29])]).double().cpu(), want[29:30], "bfloat16", "before")
    kernels.check_device_errors(certain=True)                     # nothing is wrong yet
    assert kernels.wait_probe(1 << 16) is True
    with pytest.raises(BackendError, match="gave up waiting"):
        kernels.check_device_errors()
    kernels.check_device_errors(certain=True)                     # read and cleared: all is well again
    for p in range(30, 40):                                       # recorded decode steps after the failure
        runner.cache.extend(1, p + 1)
        got = runner.step([SequenceStep(1, [tokens[p]], p, [0])]).double().cpu()
        T.check_rows(got, want[p:p + 1], "bfloat16", f"decode step at {p} after a wait ran out")
    runner.cache.close(1)

    limits = RuntimeConfig(max_seq_len=128, page_size=16, prefill_budget=16, max_running=2)
    engine = EngineHandle.load(folder, 0, config=limits, dtype="bfloat16", num_pages=16)
    stream = engine.generate(GenerateRequest(TokenIds(tokens[:20]), SamplingParams(max_tokens=8, ignore_eos=True)))
    assert engine.run_step() and engine.run_step()
    real = engine.runner.forward

    def forward_with_a_stuck_wait(batch, observe=None, carried=None):
        logits = real(batch, observe, carried)
        kernels.wait_probe(1 << 16)
        return logits

    engine.runner.forward = forward_with_a_stuck_wait
    with pytest.raises(BackendError, match="gave up waiting"):
        engine.run_step()               # the step is queued; the host looks at the error words when it reads a step's
        engine.run_step()               # tokens, which with overlapped steps is one call later
    events = list(stream.events)
    assert any(isinstance(e, Error) for e in events) and events[-1].reason == "error"
    assert engine.healthy is False and engine.metrics()["free_pages"] == 16
    kernels.check_device_errors(certain=True)


def test_dropping_a_stream_or_leaving_its_block_cancels_the_request(model_folders):
    import gc
    folder = model_folders["B"]
    limits = RuntimeConfig(max_seq_len=128, page_size=16, prefill_budget=16, max_running=3)
    engine = EngineHandle.load(folder, 0, config=limits, dtype="float32", num_pages=24)
    long = SamplingParams(max_tokens=60, ignore_eos=True)
    dropped = engine.generate(GenerateRequest(TokenIds([5, 6, 7]), long))
    kept = engine.generate(GenerateRequest(TokenIds([9, 8, 7, 6]), SamplingParams(max_tokens=5, ignore_eos=True)))
    assert isinstance(next(kept), Token)
    del dropped
    gc.collect()
    with engine.generate(GenerateRequest(TokenIds([1, 2]), long)) as left:
        assert isinstance(next(left), Token)
    events = list(kept)
    assert events[-1].reason == "length" and sum(isinstance(e, Token) for e in events) == 4
    while engine.run_step():
        pass
    metrics = engine.metrics()
    assert metrics["cancelled"] == 2 and metrics["completed"] == 1 and metrics["free_pages"] == 24
    assert [e.reason for e in left.events if isinstance(e, Finished)] == ["cancelled"]
    engine.shutdown()


@pytest.mark.parametrize("name,dtype", [("B", "float32"), ("D", "bfloat16")])
def test_a_whole_prompt_of_more_than_a_thousand_tokens_is_one_recorded_step(model_folders, name, dtype):
    """Steps of up to 2,048 rows are recorded: a prompt of 1,400 tokens as one step, then a second prompt of the same
    rounded length through the same recording, each beside a decoded token of a third request.  The last rows equal
    the plain implementation's and, in float32, those of a runner that queues every kernel, bit for bit."""
    vocab = TINY[name][0]["vocab_size"]
    reqs = list(T.requests_for(vocab, [1400, 1380, 40], seed=77).values())
    want = [plain(model_folders[name], tokens) for tokens in reqs]
    rows = {}
    for record in (True, False):
        runner = runner_for(model_folders[name], name, dtype, pages=3 * 1500 // TINY[name][1] + 8, max_seq_len=1536)
        assert runner.mixed_rows_max >= 1408
        runner.record_mixed = record
        for i in range(3):
            runner.cache.open(i + 1)
        runner.cache.extend(3, 38)
        runner.step([SequenceStep(3, reqs[2][:38], 0, [])])
        got = []
        for k, i in enumerate((0, 1)):
            n = len(reqs[i])
            runner.cache.extend(i + 1, n)
            runner.cache.extend(3, 39 + k)
            out = runner.step([SequenceStep(3, [reqs[2][38 + k]], 38 + k, [0]), SequenceStep(i + 1, reqs[i], 0, [n - 1])]).double().cpu()
            T.check_rows(out, torch.stack([want[2][38 + k], want[i][n - 1]]), dtype, f"prompt {i} (recorded={record})")
            got.append(out)
        if record:
            fixed = [key for key in runner._records if len(key) == 5 and key[0] >= 1408]
            assert len(fixed) == 1 and runner.recorded_steps >= 2           # both long steps through one recording
        rows[record] = torch.cat(got)
    if dtype == "float32":
        assert torch.equal(rows[True], rows[False])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_recorded_decode_steps_across_classes_of_context_length(model_folders, dtype):
    """Three requests decode from 480, 700 and 20 tokens of context until the first has passed 1,024: steps are
    recorded once per (padded batch, class of context length), so contexts that cross 512, 1,024 and the
    batch's changing make-up (all three, two of them, one alone) make several recordings, some made in the
    middle of the run, with attention split counts planned for the class and block tables of 128 pages.
    Every step's logits equal the plain implementation's; in float32 the recorded run equals, bit for bit,
    a run that queues every kernel."""
    name = "D"
    folder = model_folders[name]
    vocab = TINY[name][0]["vocab_size"]
    starts = {"r0": 480, "r1": 700, "r2": 20}
    reqs = T.requests_for(vocab, [1060, 1180, 760], seed=77)
    want = {r: plain(folder, t) for r, t in reqs.items()}
    results, keys = [], None
    for record in (True, False):
        runner = runner_for(folder, name, dtype, pages=200, max_seq_len=2048, running=4)
        runner.record_decode = record
        at = dict(starts)
        for i, (r, tokens) in enumerate(reqs.items()):
            runner.cache.open(i + 1)
            runner.cache.extend(i + 1, at[r])
            runner.step([SequenceStep(i + 1, tokens[:at[r]], 0, [])])
        ids = {r: i + 1 for i, r in enumerate(reqs)}
        rows, k = [], 0
        while at["r0"] < 1040:
            live = ["r2"] if k % 7 == 3 else (["r0", "r2"] if k % 5 == 2 else ["r0", "r1", "r2"])
            batch = []
            for r in live:
                runner.cache.extend(ids[r], at[r] + 1)
                batch.append(SequenceStep(ids[r], [reqs[r][at[r]]], at[r], [0]))
            got = runner.step(batch).double().cpu()
            T.check_rows(got, torch.stack([want[r][at[r]] for r in live]), dtype, f"step {k} at contexts {[at[r] for r in live]} (recorded={record})")
            rows.append(got)
            for r in live:
                at[r] += 1
            k += 1
        assert at["r1"] > 1024 and at["r2"] > 512
        if record:
            keys = sorted(key for key in runner._records if len(key) == 2)      # the decode steps' recordings
            assert len(keys) >= 5, keys
            assert {c for _, c in keys} == {512, 1024, 2048} and {b for b, _ in keys} == {1, 2, 4}
            assert runner._records[keys[0]].ctx.block_tables[0].shape[1] == 128
        else:
            assert not runner._records
        results.append(rows)
    if dtype == "float32":
        assert all(torch.equal(a, b) for a, b in zip(*results))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_real_vocabulary_and_a_recorded_step_beyond_2048_tokens(dtype):
    """Two layers with the sizes of a real checkpoint and its real vocabulary of 151,936: a prompt of 2,040 tokens
    in portions of 512, then twelve decoded tokens (recorded steps whose context passes 2,048).  The logits of the
    last prompt token and of every decoded token equal the plain implementation's, whose head product runs in
    slices of the vocabulary, and the arg-max kernel picks the plain arg-max (or a logit within rounding of it)."""
    from conftest import REAL_LAYERS
    from mini_rsglang_b200 import kernels
    from mini_rsglang_b200.models import config_from_dict
    from mini_rsglang_b200.models.registry import model_spec_for
    from mini_rsglang_b200.parts import Runtime
    from mini_rsglang_b200.weights.random_init import random_weights

    raw = dict(REAL_LAYERS, vocab_size=151936, max_position_embeddings=4096)
    config = config_from_dict(raw)
    spec = model_spec_for(config)
    held = torch.bfloat16 if dtype == "bfloat16" else torch.float32
    stored = random_weights(spec.weight_specs(), 33, torch.bfloat16, "cuda:0")         # a checkpoint's bfloat16 values
    tensors = {n: (t if t.dtype is torch.float32 else t.to(held)) for n, t in stored.items()}
    limits = RuntimeConfig(max_seq_len=2304, page_size=16, prefill_budget=512, max_running=2)
    runner = ModelRunner(config, tensors, Runtime(torch.device("cuda:0"), held, 16), limits, num_pages=160, spec=spec)
    prompt_len, steps = 2040, 12
    tokens = T.requests_for(raw["vocab_size"], [prompt_len + steps], seed=12)["r0"]

    # the plain implementation, part by part; the head in slices of 8,192 rows of the vocabulary
    cfg = P.PlainConfig(raw["hidden_size"], raw["intermediate_size"], 2, raw["num_attention_heads"], raw["num_key_value_heads"],
                        raw["head_dim"], raw["vocab_size"], raw["rms_norm_eps"], raw["rope_theta"], False)
    weights = stored            # on the GPU: the plain functions compute where their tensors lie, in float64
    ar = P.Arith(None)
    ids = torch.tensor(tokens, device="cuda:0")
    x = weights["model.embed_tokens.weight"][ids].double()
    positions = torch.arange(len(tokens), device="cuda:0")
    for layer in range(2):
        x = P.block(ar, cfg, weights, layer, x, positions)
    places = list(range(prompt_len - 1, prompt_len + steps))
    hidden = P.rms_norm(ar, x[places], weights["model.norm.weight"], cfg.rms_norm_eps)
    head = weights["lm_head.weight"]
    want = torch.cat([hidden @ head[a:a + 8192].double().T for a in range(0, head.shape[0], 8192)], dim=1).cpu()
    del x, hidden

    runner.cache.open(1)
    got, pos = [], 0
    for n in (512, 512, 512, prompt_len - 1536):
        runner.cache.extend(1, pos + n)
        logits = runner.step([SequenceStep(1, tokens[pos:pos + n], pos, [n - 1] if pos + n == prompt_len else [])])
        pos += n
    got.append(logits.double().cpu())
    picked = torch.empty(1, dtype=torch.int32, device="cuda:0")
    choices = []
    for p in range(prompt_len, prompt_len + steps):
        runner.cache.extend(1, p + 1)
        logits = runner.step([SequenceStep(1, [tokens[p]], p, [0])])
        kernels.argmax(logits, picked)
        choices.append(int(picked.item()))
        got.append(logits.double().cpu())
    got = torch.cat(got)
    T.check_rows(got, want, dtype, "real vocabulary")
    assert sorted(key for key in runner._records if len(key) == 2) == [(1, 2048), (1, 4096)]
    for row, choice in zip(want[1:], choices):
        best = P.greedy(row)
        allowed = 2e-5 * max(1.0, row.abs().max().item()) if dtype == "float32" else 0.02 * row.abs().max().item()
        assert choice == best or (row[best] - row[choice]).item() <= allowed
