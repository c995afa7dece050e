"""Layer by layer: `bin/trace_run --observe ID` writes what the reference's observer sees
(crates/models/src/qwen3.rs:159-229) for one request, step by step; every label is compared with the
plain implementation's tensor of the same name, in float32 and in bfloat16, for a request that comes in
portions and single tokens beside another request."""
import glob
import os

import numpy as np
import pytest
import torch

import plain_qwen3 as P
import trace_tools as T

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "D"])
def test_every_observed_layer_matches_the_plain_implementation(model_folders, tmp_path, name, dtype):
    folder = model_folders[name]
    cfg, weights = P.PlainConfig.load(folder), P.load_plain_weights(folder)
    reqs = T.requests_for(cfg.vocab_size, [40, 31], seed=77)
    watched, other = reqs["r0"], reqs["r1"]
    want = {}
    P.logits_of_sequence(cfg, weights, watched, observe=lambda label, t: want.__setitem__(label, t.double()))
    labels = ["embedding", "final_norm"] + [f"layer{i}-{part}" for i in range(cfg.num_hidden_layers) for part in
                                              ("input_norm", "q_proj", "q_norm", "q_rope", "k_rope", "v_proj", "attn", "swiglu", "output")]
    assert sorted(want) == sorted(labels)
    # the watched request: 23 tokens, 9 tokens, then one by one; the other request beside it, before it in the batch
    cuts = [23, 9] + [1] * 8
    steps, at, other_at = [], 0, 0
    for i, n in enumerate(cuts):
        entries = []
        if other_at < len(other):
            m = min(7, len(other) - other_at)
            entries.append({"id": "r1", "tokens": other[other_at:other_at + m], "want": []})
            other_at += m
        entries.append({"id": "r0", "tokens": watched[at:at + n], "want": [n - 1]})
        at += n
        steps.append({"step": i, "entries": entries, "end": []})
    assert at == len(watched)
    out = str(tmp_path / "out")
    run = T.TraceRun(folder, dtype, out, 128, extra=("--observe", "r0"))
    for step in steps:
        run.step(step, cfg.vocab_size)
    assert run.close() == 0
    for label in labels:
        parts = []
        for i, n in enumerate(cuts):
            data = np.fromfile(os.path.join(out, "observe", f"{i}.{label}.f32"), dtype="<f4")
            assert data.size % n == 0, f"{label}, step {i}: {data.size} floats for {n} tokens"
            parts.append(torch.from_numpy(data.reshape(n, -1).astype(np.float64)))
        got = torch.cat(parts)
        assert got.shape == want[label].shape, f"{label}: {tuple(got.shape)} against {tuple(want[label].shape)}"
        T.check_rows(got, want[label], dtype, f"{name} {dtype} {label}")
    assert len(glob.glob(os.path.join(out, "observe", "*.f32"))) == len(labels) * len(cuts)
