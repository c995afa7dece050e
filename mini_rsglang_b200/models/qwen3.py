"""Qwen3 dense as a composition of parts (reference: crates/models/src/qwen3.rs:44-236):
pre-norm blocks of grouped-query attention (per-head RMSNorm of q and k, rotary positions,
every key kept) and a SiLU-gated feed-forward, RMSNorm everywhere, an output head that may be
tied to the embedding.  Tensor names are the checkpoint's (crates/models/src/weights.rs:73-162)."""
from __future__ import annotations

from ..config.model_config import Qwen3Config
from ..parts.base import PartSpec
from .spec import ModelSpec, pre_norm_layer


def qwen3_spec(config: Qwen3Config) -> ModelSpec:
    c = config
    norm = PartSpec("rmsnorm", {"width": c.hidden_size, "eps": c.rms_norm_eps})
    head_norm = PartSpec("rmsnorm", {"width": c.head_dim, "eps": c.rms_norm_eps})
    mixer = PartSpec("gqa_attention", {
        "width": c.hidden_size, "num_heads": c.num_attention_heads, "num_kv_heads": c.num_key_value_heads,
        "head_dim": c.head_dim, "q_norm": head_norm, "k_norm": head_norm,
        "position": PartSpec("rope", {"head_dim": c.head_dim, "theta": c.rope_theta})})
    feed_forward = PartSpec("swiglu", {"width": c.hidden_size, "inner": c.intermediate_size,
                                       "activation": c.hidden_act})
    layers = [pre_norm_layer(f"model.layers.{i}", norm, mixer, norm, feed_forward) for i in range(c.num_hidden_layers)]
    table = {"vocab": c.vocab_size, "width": c.hidden_size}
    tied = "model.embed_tokens.weight" if c.tie_word_embeddings else None
    return ModelSpec(vocab_size=c.vocab_size, width=c.hidden_size,
                     embedding=PartSpec("token_embedding", table), embedding_prefix="model.embed_tokens",
                     layers=layers, final_norm=norm, final_norm_prefix="model.norm",
                     head=PartSpec("linear_head", dict(table, tied_to=tied)), head_prefix="lm_head",
                     ignorable_weights=("lm_head.weight",) if c.tie_word_embeddings else ())
