"""A model as data: what a spec builds, and what it refuses, without a device."""
import pytest
from conftest import TINY_A, TINY_B

from mini_rsglang_b200 import InvalidRequest
from mini_rsglang_b200.models import config_from_dict
from mini_rsglang_b200.models.registry import model_spec_for
from mini_rsglang_b200.models.spec import LayerSpec, ModelSpec, RunEntry, pre_norm_layer
from mini_rsglang_b200.parts import BLOCKS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, POSITION_ENCODINGS, PartSpec


def test_every_kind_of_part_has_a_registry_with_the_engines_kinds():
    assert "token_embedding" in EMBEDDINGS.entries and "linear_head" in HEADS.entries
    assert "rmsnorm" in NORMS.entries and "gqa_attention" in MIXERS.entries and "swiglu" in FEED_FORWARDS.entries
    assert "pre_norm" in BLOCKS.entries and {"rope", "none"} <= set(POSITION_ENCODINGS.entries)
    with pytest.raises(InvalidRequest, match="unknown embedding kind"):
        EMBEDDINGS.get("no_such_embedding")
    with pytest.raises(InvalidRequest, match="registered already"):
        NORMS.register("rmsnorm", object)


@pytest.mark.parametrize("raw", [TINY_A, TINY_B])
def test_qwen3_spec_names_the_checkpoints_tensors(raw):
    config = config_from_dict(raw)
    spec = model_spec_for(config)
    names = [s.name for s in spec.weight_specs()]
    per_layer = ["input_layernorm.weight", "self_attn.q_proj.weight", "self_attn.k_proj.weight", "self_attn.v_proj.weight",
                 "self_attn.o_proj.weight", "self_attn.q_norm.weight", "self_attn.k_norm.weight",
                 "post_attention_layernorm.weight", "mlp.gate_proj.weight", "mlp.up_proj.weight", "mlp.down_proj.weight"]
    want = ["model.embed_tokens.weight"] + [f"model.layers.{i}.{leaf}" for i in range(config.num_hidden_layers) for leaf in per_layer]
    want += ["model.norm.weight"] + ([] if config.tie_word_embeddings else ["lm_head.weight"])
    assert names == want
    assert len(spec.run_order) == config.num_hidden_layers and all(e.cache_of is None for e in spec.run_order)


def test_a_layer_must_give_exactly_the_parts_that_its_block_kind_arranges():
    norm = PartSpec("rmsnorm", {"width": 8, "eps": 1e-6})
    ff = PartSpec("swiglu", {"width": 8, "inner": 16})
    table = {"vocab": 10, "width": 8}

    def model(layer):
        return ModelSpec(vocab_size=10, width=8, embedding=PartSpec("token_embedding", table), embedding_prefix="e",
                         layers=[layer], final_norm=norm, final_norm_prefix="n",
                         head=PartSpec("linear_head", dict(table, tied_to="e.weight")), head_prefix="h")

    with pytest.raises(InvalidRequest, match=r"missing \['mixer'\]"):
        model(LayerSpec("l", "pre_norm", {"norm1": norm, "norm2": norm, "feed_forward": ff})).build_parts()
    with pytest.raises(InvalidRequest, match=r"unknown \['norm3'\]"):
        model(LayerSpec("l", "pre_norm", {"norm1": norm, "mixer": norm, "norm2": norm, "feed_forward": ff, "norm3": norm})).build_parts()
    with pytest.raises(InvalidRequest, match="unknown block kind"):
        model(LayerSpec("l", "no_such_block", {})).build_parts()


def test_run_order_may_name_a_layer_twice_and_borrow_an_earlier_cache_only():
    spec = model_spec_for(config_from_dict(TINY_A))
    twice = ModelSpec(**{**spec.__dict__, "run_order": [RunEntry(0), RunEntry(1), RunEntry(0, cache_of=0)]})
    assert [e.layer for e in twice.run_order] == [0, 1, 0]
    for order in ([RunEntry(0, cache_of=0)], [RunEntry(0), RunEntry(1, cache_of=1)], [RunEntry(0), RunEntry(1, cache_of=0), RunEntry(0, cache_of=1)],
                  [RunEntry(5)]):
        with pytest.raises(InvalidRequest):
            ModelSpec(**{**spec.__dict__, "run_order": order})


def test_pre_norm_layer_uses_the_usual_tensor_roots():
    norm = PartSpec("rmsnorm", {"width": 8, "eps": 1e-6})
    layer = pre_norm_layer("model.layers.3", norm, norm, norm, norm, mixer_name="mixer")
    assert layer.block == "pre_norm" and layer.names["mixer"] == "mixer" and layer.names["norm1"] == "input_layernorm"
