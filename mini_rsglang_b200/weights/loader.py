"""Binding a checkpoint to the tensors a model asks for, by name.

One pass collects everything that is wrong (missing names, names nobody asked for, shapes
that differ) and raises one `InvalidRequest` that lists all of it, where the reference
stops at the first (crates/models/src/weights.rs:45-60; crates/models/src/qwen3.rs:48-58,
128-133).  Files: `model.safetensors`, or the shards that `model.safetensors.index.json`
names, each a bare `*.safetensors` file name (weights.rs:21-39)."""
from __future__ import annotations

import json
import os
from typing import Iterable

import torch

from ..errors import InvalidRequest
from .safetensors_io import SafetensorsFile, StoredTensor
from .spec import WeightSpec

_FLOATS = ("F64", "F32", "F16", "BF16")
_INTS = ("I64", "I32", "I16", "I8", "U8")


def checkpoint_files(folder: str) -> list[str]:
    index = os.path.join(folder, "model.safetensors.index.json")
    if os.path.exists(index):
        with open(index) as f:
            try:
                weight_map = json.load(f)["weight_map"]
                assert isinstance(weight_map, dict)
            except (json.JSONDecodeError, KeyError, AssertionError, TypeError):
                raise InvalidRequest("safetensors index missing weight_map") from None
        files = set()
        for file in weight_map.values():
            if (not isinstance(file, str) or os.path.basename(file) != file
                    or not file.endswith(".safetensors")):
                raise InvalidRequest("shard must be a local safetensors filename")
            files.add(file)
        return [os.path.join(folder, f) for f in sorted(files)]
    single = os.path.join(folder, "model.safetensors")
    if not os.path.exists(single):
        raise InvalidRequest(f"{folder}: neither model.safetensors nor model.safetensors.index.json")
    return [single]


def open_checkpoint(folder: str) -> dict[str, StoredTensor]:
    stored: dict[str, StoredTensor] = {}
    for path in checkpoint_files(folder):
        for name, tensor in SafetensorsFile(path).tensors.items():
            if name in stored:
                raise InvalidRequest(f"duplicate tensor {name}")
            stored[name] = tensor
    return stored


def held_dtype(role: str, engine_dtype: torch.dtype) -> torch.dtype:
    if role == "vector":
        return torch.float32
    if role == "int_table":
        return torch.int32
    return engine_dtype


def load_weights(folder: str, specs: Iterable[WeightSpec], engine_dtype: torch.dtype,
                 device: torch.device | str = "cpu", ignorable: Iterable[str] = ()) -> dict[str, torch.Tensor]:
    """Read every tensor of `specs` from the checkpoint in `folder`.

    `engine_dtype` is bfloat16 or float32.  Floating tensors stored as bfloat16 stay
    bfloat16 when serving and are widened (exactly) on the 32-bit path; float16 and float32
    matrices are converted to the engine's dtype; vectors are held in float32 and integer
    tables as int32.  `ignorable` names tensors that may be in the files without being used
    (the reference skips `lm_head.weight` of a tied model, weights.rs:49-51)."""
    specs = list(specs)
    stored = open_checkpoint(folder)
    wanted = {s.name: s for s in specs}
    if len(wanted) != len(specs):
        raise InvalidRequest("internal: a model asked twice for the same tensor name")
    missing = [name for name in wanted if name not in stored]
    ignorable = set(ignorable)
    unexpected = [name for name in stored if name not in wanted and name not in ignorable]
    wrong = []
    for name, spec in wanted.items():
        if name not in stored:
            continue
        t = stored[name]
        if tuple(t.shape) != tuple(spec.shape):
            wrong.append(f"{name}: shape {list(t.shape)}, expected {list(spec.shape)}")
        elif spec.role == "int_table" and t.dtype not in _INTS:
            wrong.append(f"{name}: dtype {t.dtype}, expected an integer table")
        elif spec.role != "int_table" and t.dtype not in _FLOATS:
            wrong.append(f"{name}: unsupported weight dtype {t.dtype}")
    if missing or unexpected or wrong:
        parts = [f"checkpoint {folder} does not match the model:"]
        if missing:
            parts.append(f"  missing weights ({len(missing)}): " + ", ".join(sorted(missing)))
        if unexpected:
            parts.append(f"  unexpected weights ({len(unexpected)}): " + ", ".join(sorted(unexpected)))
        if wrong:
            parts.append(f"  wrong shape or dtype ({len(wrong)}): " + "; ".join(sorted(wrong)))
        raise InvalidRequest("\n".join(parts))
    out = {}
    for name, spec in wanted.items():
        tensor = stored[name].read()
        out[name] = tensor.to(device=device, dtype=held_dtype(spec.role, engine_dtype))
    return out
