"""Grouped-query attention over the paged cache, with optional per-head q/k norms and a
position encoding (reference: crates/models/src/qwen3.rs:178-202).

One projection gives q, k and v (the three matrices are concatenated by rows when bound);
one kernel applies the head norms and the rotation and writes k and v into the cache pages;
attention reads the cache through the request's block table; one projection brings the
heads back to the model width."""
from __future__ import annotations

import os
from dataclasses import dataclass

import numpy as np
import torch

from .. import kernels
from ..errors import InvalidRequest
from ..weights.spec import WeightSpec
from .base import MIXERS, NORMS, POSITION_ENCODINGS, KVNeed, Mixer, PartSpec, Prenormed, StepFacts, observing
from .linear import few_rows, linear


@dataclass
class TileLists:
    """A step's attention tiles as the host planned them: `narrow` for the kernels for few rows, `wide` for the
    others, entries (sequence, first row of the step, tokens, share word).  For a step with fixed shapes
    `narrow_cap` and `wide_cap` are the rows of the two lists on the device (filled up with entries of no
    tokens, which the kernels skip); 0 there: the list is empty and its kernel is not launched."""

    narrow: list
    wide: list
    longest_narrow: int
    shared: bool
    narrow_cap: int = 0
    wide_cap: int = 0

    def signature(self) -> tuple:
        return (self.narrow_cap, self.wide_cap, self.shared)

    def words(self) -> np.ndarray:
        """The lists as the int32 words of the device copy of a step with fixed shapes."""
        out = np.zeros((self.narrow_cap + self.wide_cap, 4), dtype=np.int32)
        if self.narrow:
            out[:len(self.narrow)] = self.narrow
        if self.wide:
            out[self.narrow_cap:self.narrow_cap + len(self.wide)] = self.wide
        return out.reshape(-1)


def attention_tile_lists(facts: StepFacts, group: int, wide_rows: int, kv_heads: int = 1, window: int = 0,
                         key_block: int = 128, sms: int = 1) -> TileLists:
    """Cuts the step's sequences into tiles for the tensor-core kernels, on the host: sequences with few
    query rows (decoded tokens, short portions) go to the kernels for few rows in tiles of
    16 // group tokens, the others in tiles of wide_rows // group tokens, those with the most
    keys first.  The lists are kept in `facts.plans` for the other layers of the step.

    The tcgen05 kernel for wide tiles takes two tiles of rows a CTA and one CTA an SM.  A short
    portion (a slice of a long prompt under the token budget) makes fewer CTAs than the GPU has
    SMs.  Then, measured with 512 tokens behind 3,584 cached ones and 8 key/value heads (78 us as
    64 CTAs): entries with at least 8 blocks of 128 keys are cut into shares of their keys, whose
    sums a second kernel merges; shorter ones into entries of one tile (68 us as 128 CTAs; a CTA
    with one tile has no partner on the tensor cores, so this pays only while SMs would idle).
    `key_block` is the kernel's block of keys and `sms` the device's multiprocessors, as the kernel's
    library and the device state them."""
    key = (group, wide_rows, kv_heads, window, key_block)
    if key in facts.plans:
        return facts.plans[key]
    narrow_tokens = kernels.MMA_ROWS_NARROW // group
    tensor_core = wide_rows == kernels.PREFILL_TC_ROWS
    tiles = kernels.PREFILL_TC_TILES if tensor_core else 1            # tiles of an entry; a tile holds whole tokens
    wide_tokens = tiles * (wide_rows // tiles // group)
    real = len(facts.start_pos)
    lengths = [facts.q_start[i + 1] - facts.q_start[i] for i in range(real)]
    narrow, found = [], []
    longest_narrow = 0
    for i, n in enumerate(lengths):
        first = facts.q_start[i]
        if narrow_tokens >= 1 and n <= narrow_tokens:
            narrow.append((i, first, n, 0))
            longest_narrow = max(longest_narrow, facts.start_pos[i] + n)
            continue
        for start in range(0, n, wide_tokens):
            tokens = min(wide_tokens, n - start)
            begin = facts.start_pos[i] + start                           # position of the entry's first token
            first_key = max(0, begin - window + 1) if window else 0
            blocks = -(-(begin + tokens) // key_block) - first_key // key_block
            found.append((i, first + start, tokens, begin, blocks))
    # CTAs an entry may become.  Beside decoded tokens the kernel for few rows runs at the same time and wants SMs
    # of its own: the wide entries then share WIDE_SHARE_BESIDE_NARROW of them.
    room = int(sms * WIDE_SHARE_BESIDE_NARROW) if narrow else sms
    spare = room // max(len(found) * kv_heads, 1) if tensor_core else 1
    wide = []
    shared = False
    if tensor_core and tiles == 2 and spare < 2 and len(found) * kv_heads <= room and not window and PAIR_FAR_TILES:
        # One round of CTAs, more than half the SMs: what is left to gain is their balance.  The tiles of a portion
        # walk 1, 2, 3, ... blocks of keys more than the first, and a CTA holds two tiles: the first with the last,
        # the second with the last but one, and so on, so that every CTA has the same work; the early tile is done
        # after a few blocks and the late one walks on alone.  The entry's fourth number carries the tokens between
        # its tiles (<< 16).  Measured alone, neighbours against pairs: 2,048 tokens of 16 query heads (128 CTAs)
        # 42.9 against 39.9 us, 512 tokens of 40 heads (88 CTAs) 19.9 against 18.8 us, 1,024 tokens of 32 heads
        # (128 CTAs) 26.5 against 26.1 us.  With more CTAs than SMs the rounds balance themselves and the pairs lose,
        # since a tile without a partner uses the tensor cores half (2,048 tokens of 32 heads, 256 CTAs: 49.6 against
        # 64.5 us; 8,192 tokens: 494 against 683 us), so neighbours stay together there.
        per_tile = wide_tokens // 2
        for i, n in enumerate(lengths):
            if narrow_tokens >= 1 and n <= narrow_tokens:
                continue
            count = -(-n // per_tile)
            first, begin = facts.q_start[i], facts.start_pos[i]
            if count < 4 or count * per_tile >= 1 << 15:
                wide += [(i, f, t, 0, 2 * b) for (j, f, t, p, b) in found if j == i]
                continue
            for a in range(count // 2):
                b = count - 1 - a
                last = min(per_tile, n - b * per_tile)
                blocks_a = -(-(begin + (a + 1) * per_tile) // key_block)
                blocks_b = -(-(begin + b * per_tile + last) // key_block)
                wide.append((i, first + a * per_tile, per_tile + last, ((b - a - 1) * per_tile) << 16, 1.2 * blocks_b + 0.8 * blocks_a))
            if count % 2:
                a = count // 2
                wide.append((i, first + a * per_tile, per_tile, 0, 1.2 * -(-(begin + (a + 1) * per_tile) // key_block)))
        wide.sort(key=lambda t: -t[4])          # by the time they take, in blocks of two tiles
        wide = [t[:4] for t in wide]
        found = []
    for i, first, tokens, begin, blocks in found:
        shares = min(spare, blocks // 4, 255) if spare >= 2 else 1
        if shares >= 2:
            shared = True
            wide += [(i, first, tokens, s | shares << 8, begin) for s in range(shares)]
        elif spare >= 2 and tokens > wide_tokens // 2 >= 1:
            half = wide_tokens // 2
            wide += [(i, first, half, 0, begin), (i, first + half, tokens - half, 0, begin + half)]
        else:
            wide.append((i, first, tokens, 0, begin))
    if found:
        wide.sort(key=lambda t: -t[4])      # a tile late in a long request walks the most keys: start it first (stable:
        wide = [t[:4] for t in wide]        # the shares of an entry stay together and in their order)
    lists = TileLists(narrow, wide, longest_narrow, shared)
    if facts.padded_sequences:              # fixed shapes: the device lists have a length that many steps share
        lists.narrow_cap = facts.padded_sequences if narrow else 0
        lists.wide_cap = max(16, 1 << (len(wide) - 1).bit_length()) if wide else 0
    facts.plans[key] = lists
    return lists


def plan_attention_tiles(ctx, group: int, wide_rows: int, kv_heads: int = 1, window: int = 0, key_block: int = 128,
                         sms: int = 1):
    """The step's tile lists on the device: (narrow tiles, wide tiles, longest context of a narrow tile,
    whether wide tiles share their keys), None for an empty list.  The plan is kept in the context for the
    other layers of the step.  A step of single decoded tokens brings its own list; a step with fixed shapes
    finds the lists where the step function copied them (`ctx.plan_views`), at addresses that stay."""
    plans = ctx.__dict__.setdefault("_attention_plans", {})
    key = (group, wide_rows, kv_heads, window, key_block)
    if key in plans:
        return plans[key]
    narrow_tokens = kernels.MMA_ROWS_NARROW // group
    if ctx.decode_tiles is not None and narrow_tokens >= 1:     # single tokens: the step's own tile list
        plans[key] = (ctx.decode_tiles, None, ctx.max_context_len, False)
        return plans[key]
    facts = ctx.facts
    if facts is None:
        real = ctx.real_sequences or ctx.num_sequences
        facts = StepFacts(ctx.host_q_start[:real + 1], ctx.host_start_pos[:real], ctx.max_context_len)
    lists = attention_tile_lists(facts, group, wide_rows, kv_heads, window, key_block, sms)
    if ctx.plan_views is not None:
        both = ctx.plan_views[key]
        plans[key] = (both[:lists.narrow_cap] if lists.narrow_cap else None, both[lists.narrow_cap:] if lists.wide_cap else None,
                      ctx.max_context_len, lists.shared)
        return plans[key]
    device = ctx.positions.device
    both = torch.tensor(lists.narrow + lists.wide, dtype=torch.int32).view(-1, 4).pin_memory().to(device, non_blocking=True)
    plans[key] = (both[:len(lists.narrow)] if lists.narrow else None, both[len(lists.narrow):] if lists.wide else None,
                  min(lists.longest_narrow, ctx.max_context_len), lists.shared)
    return plans[key]


def choose_splits(tiles: int, nkv: int, longest_context: int, sms: int, resident: int = 2, clusters=None) -> int:
    """CTAs per tile in the kernels for few rows.  Powers of two (2, 4, 8 or 16 shares run as one thread-block
    cluster and merge through distributed shared memory), every share with at least two 64-key blocks, all CTAs
    resident at once (`resident` per SM), at most 8 shares (16 for a single request with a long context); with
    many keys and few requests any count that fills seven eighths of the slots; one share fewer (which then meet
    through memory) where clusters of 8 or 16 would take nearly all that the GPU holds at once.  `clusters(size)`:
    how many clusters of that size the GPU holds at once (None: not asked).

    Measured on a B200 with 8 key/value heads of 128, contexts of 4,096 and 16,384, 1 to 16 requests, the kernel
    alone and in decode steps.  With few keys in all (up to about 75 MB a layer) the kernel is bound by its start and
    its merge, and the fewest shares that give every SM a CTA are best (4 requests at 4,096: a decode step takes
    3.89 ms with 4 shares, 4.13 ms with 8); with more keys it is bound by memory and wants two CTAs an SM (8
    requests: 4.23 ms with 4 shares, 4.49 ms with 2).  More CTAs than slots, or clusters of 16 for more than one
    request, cost 9 to 12 us a layer (2 requests at 4,096: 13.7 us with 8 shares, 24.4 us with 16; 6 requests:
    22.2 us with 4, 30.8 us with 8; 12 requests: 36.3 us with 2, 45.5 us with 4; a decode step at batch 2 went from
    4.04 to 3.66 ms when the count stopped being rounded up past the slots).  The GPU holds 33 clusters of 8; with 4
    requests 8 shares are 32 of them, and inside a decode step (not alone) they come to stand late, between the
    products before and after: 12 layers at a context of 16,384 take 1.970 ms a step with 8 shares, 1.709 ms with 7,
    1.742 with 6, 1.849 with 4; at 4,096 1.483, 1.376, 1.395 and 1.399 ms.  With 3 requests in the same recording
    7 shares cost 2% (1.642 against 1.599 ms).  One or two requests with long contexts want more shares than a
    cluster has, so many that seven eighths of the slots are taken (counts that are no cluster meet through memory,
    which the long walks pay for): 12 layers at a context of 36,000, one request 1.608 ms a step with 16 shares,
    1.524 with 32; two requests 1.914 ms with 8 shares, 1.757 with 18 (16, as clusters of 16: 2.062)."""
    if os.environ.get("MRS_DECODE_SPLITS"):           # the variable: for measuring other counts
        return int(os.environ["MRS_DECODE_SPLITS"])
    blocks = -(-longest_context // 64)
    slots = sms * resident
    pairs = max(tiles * nkv, 1)
    most = max(1, min(8, blocks // 2))
    if pairs * 16 <= slots // 2 and blocks // 16 >= 16:
        most = 16
    splits = 1
    if pairs * blocks <= FEW_KEYS_BLOCKS:           # few keys: stop as soon as (nearly) every SM has a CTA
        while splits * 2 <= most and pairs * splits < (85 * sms) // 100 and pairs * splits * 2 <= slots:
            splits *= 2
    else:                                           # many keys: as many resident CTAs as there are slots
        while splits * 2 <= most and pairs * splits * 2 <= slots:
            splits *= 2
        filling = min(blocks // 2, (slots * 7 // 8) // pairs, 64)
        if filling >= 8:                            # few requests with long contexts: any count that fills the GPU
            splits = filling
    if clusters is not None and splits >= 8:
        room = clusters(splits)
        if room and pairs * 5 > room * 4:           # more than four fifths of the clusters that fit at once
            splits -= 1
    return splits


FEW_KEYS_BLOCKS = 2300      # 64-key blocks over all (tile, key/value head) pairs: about 75 MB of keys and values at heads of 128


def tile_plan_arguments(d: int, group: int, page_size: int, nkv: int, window: int, device) -> tuple:
    """What the planner is asked for an attention of these sizes (bfloat16, head size a multiple of 16): rows of
    a wide tile and the block of keys as the kernel that will run states them."""
    sms = kernels.sm_count(device)
    if kernels.attention_prefill_tc_supported(d, group, page_size):
        return (group, kernels.PREFILL_TC_ROWS, nkv, window, kernels.attention_prefill_tc_key_block(d), sms)
    return (group, kernels.MMA_ROWS_WIDE, nkv, window, 128, sms)


def paged_attention(q, cache, ctx, out, nq: int, nkv: int, d: int, window: int) -> None:
    """Attention of this step's queries over their requests' cached keys and values.  bfloat16
    with a head size that is a multiple of 16 runs on the tensor cores: decoded tokens and short
    portions through the kernels for few rows (fed by bulk tensor copies when the head size is a
    multiple of 64), longer portions through the tcgen05 kernel (head sizes 64 and 128) or the
    mma.sync kernel (the others).  The 32-bit path, odd head sizes and very wide groups take the
    CUDA-core kernel."""
    table = ctx.block_tables[cache.group]
    group = nq // nkv
    if q.dtype is not torch.bfloat16 or not kernels.attention_mma_supported(d, group):
        kernels.attention_simt(q, cache.k, cache.v, ctx.positions, ctx.seq_of_token, table, out, nq, nkv, d, window)
        return
    page_size = cache.k.shape[2]
    sms = kernels.sm_count(q.device)
    tensor_core_rows = kernels.attention_prefill_tc_supported(d, group, page_size)
    narrow, wide, longest, shared = plan_attention_tiles(ctx, *tile_plan_arguments(d, group, page_size, nkv, window, q.device))
    def few_rows():
        if kernels.attention_decode_tma_supported(d, group, cache.k.shape[2]):
            splits = choose_splits(narrow.shape[0], nkv, longest, sms,
                                   clusters=lambda size: kernels.attention_decode_tma_resident_clusters(d, size, q.device))
            kernels.attention_decode_tma(q, cache.k, cache.v, ctx.positions, table, narrow, out, nq, nkv, d, window, splits)
        else:
            splits = choose_splits(narrow.shape[0], nkv, longest, sms)
            kernels.attention_mma_keys(q, cache.k, cache.v, ctx.positions, table, narrow, out, nq, nkv, d, window, splits)

    def many_rows():
        if tensor_core_rows:
            kernels.attention_prefill_tc(q, cache.k, cache.v, ctx.positions, table, wide, out, nq, nkv, d, window, shares=shared)
        else:
            kernels.attention_mma_rows(q, cache.k, cache.v, ctx.positions, table, wide, out, nq, nkv, d, window)

    if narrow is not None and wide is not None and SIDE_BY_SIDE:
        # Decoded tokens beside prompt portions: the two kernels touch other rows of q and out, and they want
        # other things of the GPU (the first streams keys at the memory's speed from few resident warps, the
        # second computes in a few CTAs that fill their SMs), so they run side by side on two streams, which a
        # recorded step keeps as two branches.
        main, side = torch.cuda.current_stream(), kernels.side_stream(q.device)
        side.wait_stream(main)
        with torch.cuda.stream(side):
            few_rows()
        many_rows()
        main.wait_stream(side)
        return
    if narrow is not None:
        few_rows()
    if wide is not None:
        many_rows()


SIDE_BY_SIDE = os.environ.get("MRS_ATTENTION_SIDE_BY_SIDE", "1") == "1"      # the variable: for measuring
# Continuous batching, 64 requests of 16 to 2,048 prompt tokens and 64 generated ones, portions under 512 tokens a
# step: 0.6B shape 143.7k tokens/s one kernel after the other, 159.9k side by side, 162.4k with the wide entries cut
# for a quarter of the SMs only (the same with no cutting at all); 8B shape 45.6k, 47.0k, 47.3k.
WIDE_SHARE_BESIDE_NARROW = float(os.environ.get("MRS_WIDE_SHARE", "0.25"))
PAIR_FAR_TILES = os.environ.get("MRS_PAIR_FAR_TILES", "1") == "1"      # the variable: for measuring


@MIXERS.register("gqa_attention")
class GroupedQueryAttention(Mixer):
    replayable = True      # reads the step's facts from device tensors only
    adds_to_stream = True
    takes_prenormed = True

    def __init__(self, prefix: str, width: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 position: PartSpec, q_norm: PartSpec | None = None, k_norm: PartSpec | None = None,
                 window: int = 0):
        super().__init__(prefix)
        if num_heads % num_kv_heads:
            raise InvalidRequest("query heads must be a multiple of key/value heads")
        if head_dim % 2 or head_dim > 256:
            raise InvalidRequest(f"head_dim {head_dim} must be even and at most 256")
        self.width, self.nq, self.nkv, self.d = int(width), int(num_heads), int(num_kv_heads), int(head_dim)
        self.window = int(window)
        self.position = POSITION_ENCODINGS.build(position, prefix)
        self.q_norm = NORMS.build(q_norm, f"{prefix}.q_norm") if q_norm else None
        self.k_norm = NORMS.build(k_norm, f"{prefix}.k_norm") if k_norm else None
        for norm in (self.q_norm, self.k_norm):
            if norm is not None and norm.width != self.d:
                raise InvalidRequest("a head norm must have the head's width")
        self.qkv = self.o = self.inv_freq = None
        self._plan_arguments = None        # what the tile planner is asked for this attention, found at first use

    def weight_specs(self):
        specs = [WeightSpec(self.name("q_proj.weight"), (self.nq * self.d, self.width)),
                 WeightSpec(self.name("k_proj.weight"), (self.nkv * self.d, self.width)),
                 WeightSpec(self.name("v_proj.weight"), (self.nkv * self.d, self.width)),
                 WeightSpec(self.name("o_proj.weight"), (self.width, self.nq * self.d))]
        for norm in (self.q_norm, self.k_norm):
            if norm is not None:
                specs += norm.weight_specs()
        return specs

    def cache_need(self):
        return KVNeed(self.nkv, self.d, "window" if self.window else "full", self.window)

    def bind(self, tensors, runtime):
        super().bind(tensors, runtime)
        self.qkv = torch.cat([tensors[self.name("q_proj.weight")], tensors[self.name("k_proj.weight")],
                              tensors[self.name("v_proj.weight")]], dim=0).contiguous()
        self.o = tensors[self.name("o_proj.weight")].contiguous()
        self.position.bind(tensors, runtime)
        for norm in (self.q_norm, self.k_norm):
            if norm is not None:
                norm.bind(tensors, runtime)
        if (self.q_norm and self.k_norm and self.q_norm.eps != self.k_norm.eps):
            raise InvalidRequest("q and k head norms must share one eps")
        rotation = self.position.rotation()
        if rotation is not None:          # the kernels' launchers say what they rotate; anything else is refused here, at load
            kernels.check_rotation(self.d, rotation.rotary_dim, rotation.pairing, rotation.magnitude)
        self.inv_freq = rotation.inv_freq if rotation is not None else None

    def step_signature(self, facts: StepFacts):
        """Which launches a step with these facts makes, beyond what its shapes say: the lengths of its tile lists
        and whether entries share their keys (None: no list is planned, one kernel takes every row)."""
        if self._plan_arguments is None:
            group = self.nq // self.nkv
            if self.runtime.dtype is not torch.bfloat16 or not kernels.attention_mma_supported(self.d, group):
                self._plan_arguments = ()
            else:
                self._plan_arguments = tile_plan_arguments(self.d, group, self.runtime.page_size, self.nkv, self.window,
                                                           self.o.device)
        if not self._plan_arguments:
            return None
        return attention_tile_lists(facts, *self._plan_arguments).signature()

    def forward(self, h, ctx, cache, write_cache=True, into=None):
        tokens = h.shape[0]
        q = torch.empty((tokens, self.nq * self.d), dtype=self.runtime.dtype, device=self.o.device)
        eps = self.q_norm.eps if self.q_norm else (self.k_norm.eps if self.k_norm else 0.0)
        group = cache.group
        prenormed = isinstance(h, Prenormed)
        if few_rows(h, self.qkv) and not observing(ctx) and \
                kernels.gemm_tc_qkv_heads_supported(h.scaled if prenormed else h, self.qkv, self.d):
            # few rows, heads of the size of the product's tiles: its epilogue norms, rotates and writes the cache itself
            kernels.gemm_tc_qkv_heads(
                h.scaled if prenormed else h, self.qkv, q, cache.k if write_cache else None, cache.v if write_cache else None,
                ctx.positions, ctx.slots[group] if write_cache else None, self.q_norm.weight if self.q_norm else None,
                self.k_norm.weight if self.k_norm else None, eps, self.inv_freq, self.nq, self.nkv,
                row_sums=h.row_sums if prenormed else None)
            out = torch.empty_like(q)
            paged_attention(q, cache, ctx, out, self.nq, self.nkv, self.d, self.window)
            return linear(out, self.o, into=into)
        qkv = linear(h, self.qkv)
        if observing(ctx):
            self._observe_projection(qkv, ctx)
        kernels.qk_norm_rope_store(
            qkv, q, cache.k if write_cache else None, cache.v if write_cache else None, ctx.positions,
            ctx.slots[group] if write_cache else None,
            self.q_norm.weight if self.q_norm else None, self.k_norm.weight if self.k_norm else None, eps,
            self.inv_freq, self.nq, self.nkv, self.d, cache.k.shape[2],
            rotations=self.position.rotations(ctx) if self.d in (64, 128, 256) else None)
        out = torch.empty_like(q)
        paged_attention(q, cache, ctx, out, self.nq, self.nkv, self.d, self.window)
        if observing(ctx):
            self._observe_rotated(q, out, cache, ctx, write_cache)
        return linear(out, self.o, into=into)

    # what the reference's observer sees in an attention layer (crates/models/src/qwen3.rs:190-201)
    def _observe_projection(self, qkv, ctx):
        tokens, q_width, kv_width = qkv.shape[0], self.nq * self.d, self.nkv * self.d
        q = qkv[:, :q_width].contiguous()
        ctx.observe(f"{ctx.label}-q_proj", q)
        ctx.observe(f"{ctx.label}-v_proj", qkv[:, q_width + kv_width:].contiguous())
        if self.q_norm is not None:
            q = self.q_norm.forward(q.view(tokens * self.nq, self.d)).view(tokens, q_width)
        ctx.observe(f"{ctx.label}-q_norm", q)

    def _observe_rotated(self, q, out, cache, ctx, write_cache):
        ctx.observe(f"{ctx.label}-q_rope", q)
        if write_cache:               # the rotated keys as they lie in the cache pages
            slots = ctx.slots[cache.group].long()
            page = cache.k.shape[2]
            ctx.observe(f"{ctx.label}-k_rope", cache.k[slots // page, :, slots % page].reshape(q.shape[0], self.nkv * self.d))
        ctx.observe(f"{ctx.label}-attn", out)
