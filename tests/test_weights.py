"""Weights: the safetensors container, binding by name with one error that lists everything
wrong, dtypes held, and seeded random models (reference checks: crates/models/src/weights.rs:45-60,
crates/models/src/qwen3.rs:48-58,128-133, crates/models/src/tests.rs:150-187)."""
import json
import os
import struct

import pytest
import torch
from conftest import TINY_A, TINY_B

from mini_rsglang_b200 import InvalidRequest
from mini_rsglang_b200.models import config_from_dict, model_spec_for
from mini_rsglang_b200.weights import (SafetensorsFile, load_weights, open_checkpoint, random_weights,
                                       write_random_model, write_safetensors)


def specs_of(raw):
    spec = model_spec_for(config_from_dict(raw))
    return spec, spec.weight_specs()


def rewrite(folder, change):
    """Load every tensor of the folder, let `change` edit the dict, write it back."""
    from safetensors.torch import load_file
    path = os.path.join(folder, "model.safetensors")
    tensors = load_file(path)
    change(tensors)
    write_safetensors(path, tensors)


def test_container_round_trip_and_foreign_reader(tmp_path):
    tensors = {"a": torch.randn(3, 5).bfloat16(), "b": torch.randn(7), "c": torch.arange(6, dtype=torch.int32).view(2, 3),
               "d": torch.randn(2, 2).half()}
    path = str(tmp_path / "x.safetensors")
    write_safetensors(path, tensors, metadata={"k": "v"})
    ours = SafetensorsFile(path)
    assert ours.metadata == {"k": "v"}
    from safetensors.torch import load_file
    theirs = load_file(path)
    for name, t in tensors.items():
        assert torch.equal(ours.tensors[name].read(), t) and torch.equal(theirs[name], t)


def test_container_range_errors(tmp_path):
    def build(header, data=b""):
        blob = json.dumps(header).encode()
        return struct.pack("<Q", len(blob)) + blob + data
    cases = {
        "short": b"\x01\x02",
        "header_too_long": struct.pack("<Q", 10_000) + b"{}",
        "not_json": struct.pack("<Q", 4) + b"nope",
        "range_outside": build({"t": {"dtype": "F32", "shape": [4], "data_offsets": [0, 16]}}, b"\0" * 8),
        "size_mismatch": build({"t": {"dtype": "F32", "shape": [4], "data_offsets": [0, 8]}}, b"\0" * 8),
    }
    for name, raw in cases.items():
        path = tmp_path / f"{name}.safetensors"
        path.write_bytes(raw)
        with pytest.raises(InvalidRequest):
            SafetensorsFile(str(path))


def test_random_model_is_seeded_and_has_the_stated_moments(tmp_path):
    cfg = config_from_dict(TINY_B)
    a = write_random_model(str(tmp_path / "a"), cfg, seed=5)
    b = write_random_model(str(tmp_path / "b"), cfg, seed=5)
    c = write_random_model(str(tmp_path / "c"), cfg, seed=6)
    spec, specs = specs_of(TINY_B)
    wa, wb, wc = (load_weights(f, specs, torch.float32) for f in (a, b, c))
    assert all(torch.equal(wa[k], wb[k]) for k in wa)
    assert any(not torch.equal(wa[k], wc[k]) for k in wa)
    big = wa["model.embed_tokens.weight"]
    assert abs(big.mean().item()) < 2e-3 and abs(big.std().item() - 0.02) < 2e-3
    norms = torch.cat([v.flatten() for k, v in wa.items() if "norm" in k])
    assert abs(norms.mean().item() - 1.0) < 0.02 and 0.03 < norms.std().item() < 0.07
    assert sorted(os.listdir(a)) == ["config.json", "model.safetensors"]
    # a tensor's values do not depend on which other tensors exist
    assert torch.equal(random_weights(specs[:3], 5, torch.bfloat16)[specs[2].name],
                       random_weights(specs[2:], 5, torch.bfloat16)[specs[2].name])


def test_dtypes_held(tmp_path):
    cfg = config_from_dict(TINY_A)
    spec, specs = specs_of(TINY_A)
    stored_bf16 = write_random_model(str(tmp_path / "bf16"), cfg, 1, torch.bfloat16)
    stored_f32 = write_random_model(str(tmp_path / "f32"), cfg, 1, torch.float32)
    assert {t.dtype for t in open_checkpoint(stored_bf16).values()} == {"BF16"}
    assert {t.dtype for t in open_checkpoint(stored_f32).values()} == {"F32"}
    serving = load_weights(stored_bf16, specs, torch.bfloat16, ignorable=spec.ignorable_weights)
    wide = load_weights(stored_bf16, specs, torch.float32, ignorable=spec.ignorable_weights)
    for s in specs:
        assert serving[s.name].dtype == (torch.float32 if s.role == "vector" else torch.bfloat16)
        assert wide[s.name].dtype == torch.float32
        assert torch.equal(serving[s.name].float(), wide[s.name])        # widening is exact
    full = load_weights(stored_f32, specs, torch.float32)
    name = "model.layers.0.mlp.down_proj.weight"
    assert not torch.equal(full[name], full[name].bfloat16().float())   # a 32-bit file keeps its 32 bits
    assert torch.equal(load_weights(stored_f32, specs, torch.bfloat16)["model.norm.weight"], full["model.norm.weight"])


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    cfg = config_from_dict(TINY_B)
    folder = write_random_model(str(tmp_path / "m"), cfg, 3)
    spec, specs = specs_of(TINY_B)

    def damage(t):
        del t["model.layers.1.mlp.up_proj.weight"]
        del t["model.norm.weight"]
        t["model.layers.9.extra.weight"] = torch.zeros(2)
        t["model.layers.0.self_attn.q_norm.weight"] = torch.zeros(16, dtype=torch.bfloat16)
        t["lm_head.weight"] = torch.zeros(96, 384, dtype=torch.bfloat16)
    rewrite(folder, damage)
    with pytest.raises(InvalidRequest) as e:
        load_weights(folder, specs, torch.bfloat16)
    text = str(e.value)
    assert "missing weights (2)" in text and "model.layers.1.mlp.up_proj.weight" in text and "model.norm.weight" in text
    assert "unexpected weights (1)" in text and "model.layers.9.extra.weight" in text
    assert "model.layers.0.self_attn.q_norm.weight: shape [16], expected [32]" in text
    assert "lm_head.weight: shape [96, 384], expected [384, 96]" in text


def test_tied_model_ignores_a_stored_head_but_untied_needs_it(tmp_path):
    cfg = config_from_dict(TINY_A)
    folder = write_random_model(str(tmp_path / "m"), cfg, 3)
    spec, specs = specs_of(TINY_A)
    rewrite(folder, lambda t: t.update({"lm_head.weight": t["model.embed_tokens.weight"].clone()}))
    load_weights(folder, specs, torch.bfloat16, ignorable=spec.ignorable_weights)
    with pytest.raises(InvalidRequest, match="unexpected weights"):
        load_weights(folder, specs, torch.bfloat16)


def test_integer_tensor_where_a_float_is_expected(tmp_path):
    cfg = config_from_dict(TINY_A)
    folder = write_random_model(str(tmp_path / "m"), cfg, 3)
    spec, specs = specs_of(TINY_A)
    rewrite(folder, lambda t: t.update({"model.norm.weight": torch.ones(64, dtype=torch.int32)}))
    with pytest.raises(InvalidRequest, match="unsupported weight dtype"):
        load_weights(folder, specs, torch.bfloat16, ignorable=spec.ignorable_weights)


def test_sharded_checkpoint_through_the_index(tmp_path):
    cfg = config_from_dict(TINY_A)
    folder = write_random_model(str(tmp_path / "m"), cfg, 3)
    spec, specs = specs_of(TINY_A)
    whole = load_weights(folder, specs, torch.bfloat16)
    from safetensors.torch import load_file
    tensors = load_file(os.path.join(folder, "model.safetensors"))
    names = sorted(tensors)
    parts = {"model-00001-of-00002.safetensors": names[::2], "model-00002-of-00002.safetensors": names[1::2]}
    for file, members in parts.items():
        write_safetensors(os.path.join(folder, file), {n: tensors[n] for n in members})
    os.remove(os.path.join(folder, "model.safetensors"))
    index = {"weight_map": {n: f for f, members in parts.items() for n in members}}
    with open(os.path.join(folder, "model.safetensors.index.json"), "w") as f:
        json.dump(index, f)
    sharded = load_weights(folder, specs, torch.bfloat16)
    assert all(torch.equal(whole[k], sharded[k]) for k in whole)
    # the same tensor in two shards
    write_safetensors(os.path.join(folder, "model-00002-of-00002.safetensors"),
                      {n: tensors[n] for n in parts["model-00002-of-00002.safetensors"] + [names[0]]})
    with pytest.raises(InvalidRequest, match="duplicate tensor"):
        load_weights(folder, specs, torch.bfloat16)
    index["weight_map"][names[0]] = "../evil.safetensors"
    with open(os.path.join(folder, "model.safetensors.index.json"), "w") as f:
        json.dump(index, f)
    with pytest.raises(InvalidRequest, match="local safetensors filename"):
        load_weights(folder, specs, torch.bfloat16)
