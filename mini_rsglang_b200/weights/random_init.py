"""Seeded random weights: for tests and benchmarks that have no checkpoint.

Every tensor has a stream of its own, keyed by the seed and the tensor's name, so a value
does not depend on which other tensors exist or in which order they are drawn.  Matrices
are N(0, 0.02); norm scales are 1 + N(0, 0.05) so that a forgotten or misplaced norm weight
shows in the output.  The reference has no such mode in its engine; its test scripts build
random checkpoints with another library (scripts/verify_tensor_parallel.py:61-93)."""
from __future__ import annotations

import hashlib
import os
from typing import Iterable

import torch

from .safetensors_io import write_safetensors
from .spec import WeightSpec

MATRIX_STD = 0.02
VECTOR_STD = 0.05


def _stream_seed(seed: int, name: str) -> int:
    digest = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(digest[:8], "little") & (2**63 - 1)


def random_tensor(spec: WeightSpec, seed: int, dtype: torch.dtype,
                  device: torch.device | str = "cpu") -> torch.Tensor:
    """One tensor of the seeded model.  Values drawn on the CPU and on a GPU differ (the
    generators differ); a folder written by `write_random_model` is drawn on the CPU."""
    device = torch.device(device)
    gen = torch.Generator(device=device)
    gen.manual_seed(_stream_seed(seed, spec.name))
    if spec.role == "int_table":
        return torch.randint(0, 2**15, spec.shape, generator=gen, device=device, dtype=torch.int32)
    values = torch.empty(spec.shape, dtype=torch.float32 if spec.role == "vector" else dtype, device=device)
    if spec.role == "vector":
        values.normal_(1.0, VECTOR_STD, generator=gen)
    else:
        values.normal_(0.0, MATRIX_STD, generator=gen)
    return values


def random_weights(specs: Iterable[WeightSpec], seed: int, dtype: torch.dtype,
                   device: torch.device | str = "cpu") -> dict[str, torch.Tensor]:
    return {s.name: random_tensor(s, seed, dtype, device) for s in specs}


def write_random_model(folder: str, config, seed: int, dtype: torch.dtype = torch.bfloat16) -> str:
    """Write `config.json` and `model.safetensors` of a seeded random model and return the
    folder.  `dtype` is the stored dtype of every floating tensor (bfloat16 as real
    checkpoints have it, or float32)."""
    from ..models.registry import model_spec_for

    spec = model_spec_for(config)
    os.makedirs(folder, exist_ok=True)
    config.save(folder)
    tensors = {}
    for ws in spec.weight_specs():
        t = random_tensor(ws, seed, dtype)
        tensors[ws.name] = t.to(dtype) if t.is_floating_point() else t
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors,
                      metadata={"format": "pt", "seed": seed})
    return folder
