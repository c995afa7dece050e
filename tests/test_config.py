"""Configuration and registry: keys, defaults, and every feature the reference rejects
(crates/models/src/config.rs:61-137; crates/models/src/tests.rs:1-80)."""
import copy
import json

import pytest
from conftest import TINY_A, TINY_B

from mini_rsglang_b200 import InvalidRequest, RuntimeConfig, SamplingParams
from mini_rsglang_b200.models import ARCHITECTURES, config_from_dict, load_config, model_spec_for

QWEN3_06B = dict(model_type="qwen3", architectures=["Qwen3ForCausalLM"], hidden_size=1024, intermediate_size=3072,
                 num_hidden_layers=28, num_attention_heads=16, num_key_value_heads=8, head_dim=128,
                 vocab_size=151936, max_position_embeddings=40960, rms_norm_eps=1e-6, rope_theta=1000000,
                 tie_word_embeddings=True, hidden_act="silu", eos_token_id=151645)


def test_qwen3_06b_shape_where_heads_times_head_dim_differs_from_hidden():
    cfg = config_from_dict(QWEN3_06B)
    assert cfg.num_attention_heads * cfg.head_dim == 2048 != cfg.hidden_size
    spec = model_spec_for(cfg)
    shapes = {s.name: s.shape for s in spec.weight_specs()}
    assert shapes["model.layers.0.self_attn.q_proj.weight"] == (2048, 1024)
    assert shapes["model.layers.27.self_attn.o_proj.weight"] == (1024, 2048)
    assert shapes["model.layers.3.self_attn.k_norm.weight"] == (128,)
    assert "lm_head.weight" not in shapes and spec.ignorable_weights == ("lm_head.weight",)


def test_untied_model_asks_for_a_head():
    spec = model_spec_for(config_from_dict(TINY_B))
    assert any(s.name == "lm_head.weight" and s.shape == (384, 96) for s in spec.weight_specs())


def test_sizes_come_from_config_not_code():
    a, b = config_from_dict(TINY_A), config_from_dict(TINY_B)
    for key in ("hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
                "num_key_value_heads", "head_dim", "vocab_size", "rms_norm_eps", "rope_theta", "tie_word_embeddings"):
        assert getattr(a, key) == TINY_A[key] and getattr(b, key) == TINY_B[key]
        assert getattr(a, key) != getattr(b, key)


@pytest.mark.parametrize("change, text", [
    ({"rope_scaling": {"type": "yarn", "factor": 4.0}}, "RoPE scaling"),
    ({"sliding_window": 4096}, "sliding window"),
    ({"use_sliding_window": True}, "sliding window"),
    ({"attention_bias": True}, "biased attention"),
    ({"hidden_act": "gelu"}, "non-SiLU"),
    ({"architectures": ["Qwen3MoeForCausalLM"]}, "Qwen3ForCausalLM"),
    ({"num_experts": 8}, "Qwen3ForCausalLM"),
    ({"head_dim": 258}, "head_dim"),
    ({"head_dim": 15}, "head_dim"),
    ({"num_key_value_heads": 3}, "GQA ratio"),
    ({"hidden_size": 0}, "positive"),
    ({"rms_norm_eps": 0.0}, "normalization"),
    ({"rope_theta": float("inf")}, "normalization"),
    ({"eos_token_id": 999999}, "eos_token_id"),
    ({"eos_token_id": []}, "EOS"),
    ({"vocab_size": 2**20, "hidden_size": 2**12}, "backend limits"),
])
def test_rejected_configurations(change, text):
    raw = copy.deepcopy(TINY_A)
    raw.update(change)
    with pytest.raises(InvalidRequest, match=text):
        config_from_dict(raw)


@pytest.mark.parametrize("key", ["hidden_size", "num_hidden_layers", "rms_norm_eps", "tie_word_embeddings",
                                 "hidden_act", "vocab_size", "max_position_embeddings", "model_type"])
def test_missing_required_key(key):
    raw = copy.deepcopy(TINY_A)
    del raw[key]
    with pytest.raises(InvalidRequest):
        config_from_dict(raw)


def test_unknown_model_type_lists_the_registered_ones():
    with pytest.raises(InvalidRequest, match="supported: .*qwen3"):
        config_from_dict({"model_type": "llama"})
    assert "qwen3" in ARCHITECTURES


def test_newer_spelling_of_rope_and_dtype_is_read(tmp_path):
    raw = copy.deepcopy(TINY_B)
    theta = raw.pop("rope_theta")
    raw["rope_parameters"] = {"rope_theta": theta, "rope_type": "default"}
    raw["dtype"] = "bfloat16"
    (tmp_path / "config.json").write_text(json.dumps(raw))
    cfg = load_config(str(tmp_path))
    assert cfg.rope_theta == theta and cfg.torch_dtype == "bfloat16"
    raw["rope_parameters"]["rope_type"] = "yarn"
    with pytest.raises(InvalidRequest, match="RoPE scaling"):
        config_from_dict(raw)


def test_head_dim_defaults_only_when_absent():
    raw = copy.deepcopy(TINY_A)
    del raw["head_dim"]
    assert config_from_dict(raw).head_dim == 16
    raw["hidden_size"] = 66
    with pytest.raises(InvalidRequest):
        config_from_dict(raw)


def test_eos_from_generation_config(tmp_path):
    cfg = config_from_dict(TINY_B)
    assert cfg.eos_ids() == [1, 2]
    cfg.save(str(tmp_path))
    assert load_config(str(tmp_path)).eos_ids(str(tmp_path)) == [1, 2]
    (tmp_path / "generation_config.json").write_text(json.dumps({"eos_token_id": [7, 9]}))
    assert cfg.eos_ids(str(tmp_path)) == [7, 9]
    (tmp_path / "generation_config.json").write_text(json.dumps({"eos_token_id": 100000}))
    with pytest.raises(InvalidRequest):
        cfg.eos_ids(str(tmp_path))


def test_runtime_limits_are_checked():
    RuntimeConfig().validate()
    for bad in (dict(page_size=3), dict(page_size=512), dict(max_waiting=0), dict(max_seq_len=0), dict(prefill_budget=-1)):
        with pytest.raises(InvalidRequest):
            RuntimeConfig(**bad).validate()


def test_sampling_params_are_checked():
    SamplingParams().validate()
    assert SamplingParams().is_greedy() and SamplingParams(temperature=0.7, top_k=1).is_greedy()
    assert not SamplingParams(temperature=0.7).is_greedy()
    for bad in (dict(temperature=float("nan")), dict(temperature=float("inf")), dict(temperature=-1.0), dict(top_p=0.0),
                dict(top_p=-0.1), dict(top_p=1.1), dict(top_p=float("nan")), dict(max_tokens=0), dict(top_k=0),
                dict(seed=-1)):
        with pytest.raises(InvalidRequest):
            SamplingParams(**bad).validate()
