"""What a part asks of a checkpoint: one `WeightSpec` per tensor."""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class WeightSpec:
    """`role` decides the dtype the tensor is held in and how random weights draw it:
    - "matrix": a projection or table of activations' kind; held in the engine's dtype
      (bfloat16 when serving, float32 on the 32-bit path); drawn N(0, 0.02);
    - "vector": a norm's scale; always held in float32 (widening bfloat16 is exact, a tensor
      stored in 32-bit stays so); drawn 1 + N(0, 0.05);
    - "int_table": integers; held as int32.
    `optional_skip` names a tensor that may be present but is not used (a tied head)."""

    name: str
    shape: tuple[int, ...]
    role: str = "matrix"
