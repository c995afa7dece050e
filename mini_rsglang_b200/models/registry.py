"""The one registry from an architecture's name (config.json `model_type`) to its typed
configuration and its model (reference: `ModelConfig::load` and `load_model`,
crates/models/src/model.rs:50-62, 133-145)."""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Callable

from ..config.model_config import ModelConfig, Qwen3Config
from ..errors import InvalidRequest
from .qwen3 import qwen3_spec
from .spec import ModelSpec


@dataclass(frozen=True)
class Architecture:
    config_class: type
    spec: Callable[[ModelConfig], ModelSpec]


ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(model_type: str, config_class: type, spec: Callable[[ModelConfig], ModelSpec],
                          replace: bool = False) -> None:
    if model_type in ARCHITECTURES and not replace:
        raise InvalidRequest(f"architecture {model_type!r} is registered already")
    ARCHITECTURES[model_type] = Architecture(config_class, spec)


register_architecture("qwen3", Qwen3Config, qwen3_spec)


def config_from_dict(raw: dict) -> ModelConfig:
    model_type = raw.get("model_type")
    if model_type not in ARCHITECTURES:
        raise InvalidRequest(f"unsupported model_type {model_type!r}; supported: {', '.join(sorted(ARCHITECTURES))}")
    return ARCHITECTURES[model_type].config_class.from_dict(raw)


def load_config(folder: str) -> ModelConfig:
    path = os.path.join(folder, "config.json")
    try:
        with open(path) as f:
            raw = json.load(f)
    except FileNotFoundError:
        raise InvalidRequest(f"{path}: no such file") from None
    except json.JSONDecodeError as e:
        raise InvalidRequest(f"{path}: not JSON: {e}") from None
    if not isinstance(raw, dict):
        raise InvalidRequest(f"{path}: not a JSON object")
    return config_from_dict(raw)


def model_spec_for(config: ModelConfig) -> ModelSpec:
    if config.model_type not in ARCHITECTURES:
        raise InvalidRequest(f"unsupported model_type {config.model_type!r}; supported: "
                             f"{', '.join(sorted(ARCHITECTURES))}")
    return ARCHITECTURES[config.model_type].spec(config)
