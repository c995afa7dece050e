"""Typed model configurations read from a checkpoint's config.json.

`ModelConfig` is what every architecture's configuration offers to the rest of the engine;
`Qwen3Config` holds the keys of Qwen3 dense under their config.json names and applies the
reference's checks (crates/models/src/config.rs:8-137).  No size stands in code: every
number the model uses comes from here."""
from __future__ import annotations

import json
import math
import os
from dataclasses import dataclass, fields
from typing import Any, ClassVar

from ..errors import InvalidRequest

INT32_MAX = 2**31 - 1


@dataclass
class ModelConfig:
    """Base of all typed configurations: the keys every architecture has."""

    model_type: str
    architectures: list[str]
    vocab_size: int
    max_position_embeddings: int
    eos_token_id: Any = None

    # the config.json values of `model_type` that this class reads
    MODEL_TYPES: ClassVar[tuple[str, ...]] = ()

    @classmethod
    def from_dict(cls, raw: dict) -> "ModelConfig":
        raise NotImplementedError

    def validate(self) -> None:
        raise NotImplementedError

    def to_dict(self) -> dict:
        """The configuration under its config.json key names."""
        return {f.name: getattr(self, f.name) for f in fields(self)}

    def save(self, folder: str) -> None:
        os.makedirs(folder, exist_ok=True)
        with open(os.path.join(folder, "config.json"), "w") as f:
            json.dump(self.to_dict(), f, indent=1)

    def eos_ids(self, folder: str | None = None) -> list[int]:
        """End-of-sequence ids: generation_config.json's `eos_token_id` when the folder has
        one, else config.json's; an int or a list (config.rs:155-184)."""
        value = self.eos_token_id
        if folder is not None:
            path = os.path.join(folder, "generation_config.json")
            if os.path.exists(path):
                with open(path) as f:
                    value = json.load(f).get("eos_token_id", value)
        values = value if isinstance(value, list) else [value]
        if not values:
            raise InvalidRequest("empty EOS token list")
        for v in values:
            if isinstance(v, bool) or not isinstance(v, int) or not 0 <= v < self.vocab_size:
                raise InvalidRequest("invalid eos_token_id")
        return list(values)


def _require(raw: dict, key: str, kind, what: str):
    if key not in raw or raw[key] is None:
        raise InvalidRequest(f"config.json: missing key `{key}` ({what})")
    value = raw[key]
    if kind is int:
        if isinstance(value, bool) or not isinstance(value, int):
            raise InvalidRequest(f"config.json: `{key}` must be an integer, got {value!r}")
    elif kind is float:
        if isinstance(value, bool) or not isinstance(value, (int, float)):
            raise InvalidRequest(f"config.json: `{key}` must be a number, got {value!r}")
        value = float(value)
    elif kind is bool:
        if not isinstance(value, bool):
            raise InvalidRequest(f"config.json: `{key}` must be true or false, got {value!r}")
    elif kind is str:
        if not isinstance(value, str):
            raise InvalidRequest(f"config.json: `{key}` must be a string, got {value!r}")
    return value


@dataclass
class Qwen3Config(ModelConfig):
    """Qwen3 dense (`Qwen3ForCausalLM`).  Required and optional keys as in the reference's
    serde struct (config.rs:8-47); a file that spells `rope_theta` inside `rope_parameters`
    and `dtype` for `torch_dtype` is accepted too."""

    hidden_size: int = 0
    intermediate_size: int = 0
    num_hidden_layers: int = 0
    num_attention_heads: int = 0
    num_key_value_heads: int = 0
    head_dim: int = 0
    rms_norm_eps: float = 0.0
    rope_theta: float = 0.0
    tie_word_embeddings: bool = False
    hidden_act: str = "silu"
    rope_scaling: Any = None
    sliding_window: Any = None
    use_sliding_window: bool = False
    attention_bias: bool = False
    torch_dtype: Any = None
    num_experts: int = 0

    MODEL_TYPES: ClassVar[tuple[str, ...]] = ("qwen3",)
    MAX_HEAD_DIM: ClassVar[int] = 256   # the attention kernels' limit (config.rs:101 has the same)

    @classmethod
    def from_dict(cls, raw: dict) -> "Qwen3Config":
        architectures = raw.get("architectures")
        if not isinstance(architectures, list) or not all(isinstance(a, str) for a in architectures):
            raise InvalidRequest("config.json: `architectures` must be a list of names")
        theta = raw.get("rope_theta")
        scaling = raw.get("rope_scaling")
        params = raw.get("rope_parameters")
        if isinstance(params, dict):
            if theta is None:
                theta = params.get("rope_theta")
            kind = params.get("rope_type", params.get("type", "default"))
            if kind not in (None, "default"):
                scaling = params
        if theta is None:
            raise InvalidRequest("config.json: missing key `rope_theta` (rotary base)")
        heads = _require(raw, "num_attention_heads", int, "query heads")
        hidden = _require(raw, "hidden_size", int, "model width")
        head_dim = raw.get("head_dim")
        if head_dim is None:
            if heads <= 0 or hidden % heads:
                raise InvalidRequest("config.json: no `head_dim` and hidden_size is no multiple of "
                                     "num_attention_heads")
            head_dim = hidden // heads
        cfg = cls(
            model_type=_require(raw, "model_type", str, "architecture family"),
            architectures=list(architectures),
            vocab_size=_require(raw, "vocab_size", int, "vocabulary"),
            max_position_embeddings=_require(raw, "max_position_embeddings", int, "longest context"),
            eos_token_id=raw.get("eos_token_id"),
            hidden_size=hidden,
            intermediate_size=_require(raw, "intermediate_size", int, "feed-forward width"),
            num_hidden_layers=_require(raw, "num_hidden_layers", int, "layers"),
            num_attention_heads=heads,
            num_key_value_heads=_require(raw, "num_key_value_heads", int, "key/value heads"),
            head_dim=head_dim,
            rms_norm_eps=_require(raw, "rms_norm_eps", float, "norm epsilon"),
            rope_theta=float(theta),
            tie_word_embeddings=_require(raw, "tie_word_embeddings", bool, "shared head"),
            hidden_act=_require(raw, "hidden_act", str, "activation"),
            rope_scaling=scaling,
            sliding_window=raw.get("sliding_window"),
            use_sliding_window=bool(raw.get("use_sliding_window", False)),
            attention_bias=bool(raw.get("attention_bias", False)),
            torch_dtype=raw.get("torch_dtype", raw.get("dtype")),
            num_experts=int(raw.get("num_experts", 0) or 0),
        )
        cfg.validate()
        return cfg

    def validate(self) -> None:
        if self.model_type != "qwen3" or self.architectures != ["Qwen3ForCausalLM"] or self.num_experts:
            raise InvalidRequest("only Qwen3ForCausalLM (dense, model_type qwen3) is supported, got "
                                 f"model_type {self.model_type!r}, architectures {self.architectures!r}, "
                                 f"num_experts {self.num_experts}")
        if (self.rope_scaling is not None or self.use_sliding_window
                or self.sliding_window is not None or self.attention_bias or self.hidden_act != "silu"):
            raise InvalidRequest("RoPE scaling, sliding window, biased attention, or non-SiLU "
                                 "architecture unsupported")
        sizes = (self.hidden_size, self.intermediate_size, self.num_hidden_layers,
                 self.num_attention_heads, self.num_key_value_heads, self.vocab_size,
                 self.max_position_embeddings, self.head_dim)
        if any(isinstance(v, bool) or not isinstance(v, int) or v <= 0 for v in sizes):
            raise InvalidRequest("invalid Qwen3 dimensions: every size must be a positive integer")
        if self.head_dim > self.MAX_HEAD_DIM or self.head_dim % 2:
            raise InvalidRequest(f"invalid Qwen3 dimensions: head_dim {self.head_dim} must be even "
                                 f"and at most {self.MAX_HEAD_DIM}")
        if self.num_attention_heads % self.num_key_value_heads:
            raise InvalidRequest("invalid Qwen3 dimensions or GQA ratio: num_attention_heads must be "
                                 "a multiple of num_key_value_heads")
        for v in (self.rms_norm_eps, self.rope_theta):
            if not math.isfinite(v) or v <= 0:
                raise InvalidRequest("invalid normalization or RoPE parameters")
        for a, b in ((self.num_attention_heads, self.head_dim), (self.num_key_value_heads, self.head_dim),
                     (self.vocab_size, self.hidden_size), (self.hidden_size, self.intermediate_size)):
            if a * b > INT32_MAX:
                raise InvalidRequest("model dimensions exceed backend limits")
        self.eos_ids()

    def to_dict(self) -> dict:
        out = super().to_dict()
        for key in ("rope_scaling", "sliding_window", "torch_dtype"):
            if out[key] is None:
                del out[key]
        if not out["num_experts"]:
            del out["num_experts"]
        return out
