"""Shared fixtures: the two tiny Qwen3 configurations (they differ in every size and option)
and model folders with seeded random weights, made in a temporary folder."""
import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the GPU box)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


TINY_A = dict(model_type="qwen3", architectures=["Qwen3ForCausalLM"], hidden_size=64, intermediate_size=128,
              num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=16, vocab_size=256,
              max_position_embeddings=1024, rms_norm_eps=1e-6, rope_theta=10000.0, tie_word_embeddings=True,
              hidden_act="silu", eos_token_id=0)
TINY_B = dict(model_type="qwen3", architectures=["Qwen3ForCausalLM"], hidden_size=96, intermediate_size=224,
              num_hidden_layers=3, num_attention_heads=6, num_key_value_heads=1, head_dim=32, vocab_size=384,
              max_position_embeddings=2048, rms_norm_eps=1e-5, rope_theta=1000000.0, tie_word_embeddings=False,
              hidden_act="silu", eos_token_id=[1, 2])
# a third shape: head size 48 (a step of 16 that is no power of two), width and vocabulary odd multiples
TINY_C = dict(model_type="qwen3", architectures=["Qwen3ForCausalLM"], hidden_size=72, intermediate_size=136,
              num_hidden_layers=2, num_attention_heads=3, num_key_value_heads=3, head_dim=48, vocab_size=301,
              max_position_embeddings=1024, rms_norm_eps=1e-6, rope_theta=50000.0, tie_word_embeddings=False,
              hidden_act="silu", eos_token_id=5)
# a fourth shape with heads of 128 and a feed-forward width that is a multiple of 64: the sizes at which the
# serving kernels of real checkpoints run (attention fed by bulk tensor copies, tcgen05 attention, the fused
# q/k/v and gate/up products)
TINY_D = dict(model_type="qwen3", architectures=["Qwen3ForCausalLM"], hidden_size=136, intermediate_size=192,
              num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=128, vocab_size=515,
              max_position_embeddings=2048, rms_norm_eps=1e-6, rope_theta=1000000.0, tie_word_embeddings=False,
              hidden_act="silu", eos_token_id=3)
TINY = {"A": (TINY_A, 4), "B": (TINY_B, 16), "C": (TINY_C, 8), "D": (TINY_D, 16)}   # configuration, page size used with it
# the layer sizes of a real checkpoint (Qwen3-8B: width 4096, 32 / 8 heads of 128, feed-forward 12288), two layers
# and a vocabulary that is no power of two: the sizes at which the serving kernels run in production
REAL_LAYERS = dict(model_type="qwen3", architectures=["Qwen3ForCausalLM"], hidden_size=4096, intermediate_size=12288,
                   num_hidden_layers=2, num_attention_heads=32, num_key_value_heads=8, head_dim=128, vocab_size=20011,
                   max_position_embeddings=4096, rms_norm_eps=1e-6, rope_theta=1000000.0, tie_word_embeddings=False,
                   hidden_act="silu", eos_token_id=7)
SHAPES = {**TINY, "R": (REAL_LAYERS, 16)}


@pytest.fixture(scope="session")
def real_size_folder(tmp_path_factory):
    """A model folder with the layer sizes of a real checkpoint (about 1 GB; made only for the tests that ask for it)."""
    from mini_rsglang_b200.models import config_from_dict
    from mini_rsglang_b200.weights import write_random_model

    folder = str(tmp_path_factory.mktemp("real_layers"))
    write_random_model(folder, config_from_dict(REAL_LAYERS), seed=21, dtype=torch.bfloat16)
    return folder


@pytest.fixture(scope="session")
def model_folders(tmp_path_factory):
    """Model folders of the tiny configurations: bfloat16 weights, seeds 11/12/13/14."""
    from mini_rsglang_b200.models import config_from_dict
    from mini_rsglang_b200.weights import write_random_model

    out = {}
    for i, (name, (raw, _)) in enumerate(TINY.items()):
        folder = str(tmp_path_factory.mktemp(f"tiny_{name}"))
        write_random_model(folder, config_from_dict(raw), seed=11 + i, dtype=torch.bfloat16)
        out[name] = folder
    return out
