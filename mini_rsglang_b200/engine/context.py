"""What one step knows about its batch, on the device.

All tokens of the step are one flat batch of `num_tokens` rows; a request's rows are
contiguous.  The reference uploads the same facts as six arrays
(`ids, positions, sequences, slots, table, last_rows`, crates/kernels/src/lib.rs:407-474);
here they are slices of one int32 buffer, copied in one transfer."""
from __future__ import annotations

from dataclasses import dataclass, field

import torch

from ..parts.base import StepFacts


@dataclass
class StepContext:
    num_tokens: int
    num_sequences: int
    token_ids: torch.Tensor            # [T] int32
    positions: torch.Tensor            # [T] int32  absolute position of each token in its request
    seq_of_token: torch.Tensor         # [T] int32  row of the block tables
    q_start: torch.Tensor              # [B + 1] int32  first row of each sequence
    context_len: torch.Tensor          # [B] int32  tokens of the sequence in the cache after this step
    state_slots: torch.Tensor          # [B] int32  state slot of each sequence
    want_rows: torch.Tensor | None     # [R] int32  rows whose logits are asked for
    block_tables: list[torch.Tensor]   # per group: [B, W_g] int32, -1 where a page was given back
    slots: list[torch.Tensor]          # per group: [T] int32  page * page_size + offset to write
    # host copies for planning launches and for parts written in Python
    host_q_start: list[int] = field(default_factory=list)
    host_start_pos: list[int] = field(default_factory=list)
    host_state_slots: list[int] = field(default_factory=list)
    max_query_len: int = 0
    max_context_len: int = 0
    fresh: list[bool] = field(default_factory=list)   # the sequence starts at position 0 in this step
    # when every sequence brings one token: [B, 4] int32 attention tiles (sequence, row, 1, 0), zeros for padding
    decode_tiles: torch.Tensor | None = None
    real_sequences: int = 0            # sequences that are not padding (padding rows come last)
    want_every_row: bool = False       # `want_rows` is 0, 1, ..., T - 1
    # Layer-by-layer inspection (the reference's observer, crates/models/src/qwen3.rs:159-229): when set, the
    # model calls observe(label, tensor [T, width]) with what the reference's observer sees under the same
    # labels, and the parts take the kernels that leave those tensors (no product with a fused epilogue).
    observe: object = None
    label: str = ""                    # the running layer's label ("layer3"), set by the model while observing
    # what the parts of one step share (the rotations' cosines and sines); the model empties it when a step begins
    shared: dict = field(default_factory=dict)
    # A step with fixed shapes (recorded once, replayed with other contents): the host's facts of the running
    # step, and for every plan that `facts.plans` holds the device copy of its words, at an address that stays.
    facts: StepFacts | None = None
    plan_views: dict | None = None
    layout_words: int = 0              # int32 words of the step's layout in its staging buffer (the plans follow them)
