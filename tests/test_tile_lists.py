"""The host's plan of a step's attention tiles (`parts/attention.py: attention_tile_lists`): every row of every
sequence in exactly one tile (or in every share of one), few rows in narrow tiles, the caps of a step with
fixed shapes."""
import random

import pytest

from mini_rsglang_b200 import kernels
from mini_rsglang_b200.parts.attention import attention_tile_lists
from mini_rsglang_b200.parts.base import StepFacts


def facts_of(lengths, starts, padded=(0, 0)):
    q_start = [0]
    for n in lengths:
        q_start.append(q_start[-1] + n)
    return StepFacts(q_start, list(starts), max(s + n for s, n in zip(starts, lengths)), padded[0], padded[1])


@pytest.mark.parametrize("group,wide_rows,sms", [(4, kernels.PREFILL_TC_ROWS, 148), (2, kernels.PREFILL_TC_ROWS, 148),
                                                 (1, 64, 1), (8, kernels.PREFILL_TC_ROWS, 16), (5, kernels.PREFILL_TC_ROWS, 148),
                                                 (3, 64, 1)])
def test_every_row_lies_in_one_tile(group, wide_rows, sms):
    rng = random.Random(group * 1000 + sms)
    for _ in range(50):
        n = rng.randint(1, 9)
        lengths = [rng.choice([1, 1, 2, 3, 17, 64, 200, 513, 1500, 2048]) for _ in range(n)]
        starts = [rng.choice([0, 0, 5, 700, 4000]) for _ in range(n)]
        facts = facts_of(lengths, starts)
        lists = attention_tile_lists(facts, group, wide_rows, 8, 0, 128, sms)
        assert attention_tile_lists(facts, group, wide_rows, 8, 0, 128, sms) is lists        # kept for the other layers
        covered = [0] * facts.q_start[-1]
        narrow_tokens = kernels.MMA_ROWS_NARROW // group
        for seq, first, tokens, share in lists.narrow:
            assert share == 0 and 0 < tokens <= narrow_tokens and tokens == lengths[seq]
            for r in range(first, first + tokens):
                covered[r] += 1
        by_share = {}
        for seq, first, tokens, share in lists.wide:
            per_tile = wide_rows // 2 // group if wide_rows == kernels.PREFILL_TC_ROWS else wide_rows // group
            assert 0 < tokens <= (2 * per_tile if wide_rows == kernels.PREFILL_TC_ROWS else per_tile)
            assert facts.q_start[seq] <= first and first + tokens <= facts.q_start[seq + 1]
            count, gap = (share >> 8) & 0xFF, share >> 16
            if count:
                assert gap == 0
                by_share.setdefault((seq, first, tokens, count), []).append(share & 0xFF)
            elif gap:                       # two tiles that are no neighbours: `gap` tokens of the request between them
                assert wide_rows == kernels.PREFILL_TC_ROWS and tokens > per_tile
                assert first + per_tile + gap + tokens - per_tile <= facts.q_start[seq + 1]
                for r in list(range(first, first + per_tile)) + list(range(first + per_tile + gap, first + gap + tokens)):
                    covered[r] += 1
            else:
                for r in range(first, first + tokens):
                    covered[r] += 1
        for (seq, first, tokens, count), indices in by_share.items():
            assert indices == list(range(count)) and lists.shared                           # all shares, in order
            for r in range(first, first + tokens):
                covered[r] += 1
        assert covered == [1] * len(covered)


def test_fixed_shapes_give_caps_that_hold_the_lists_and_words_in_their_places():
    facts = facts_of([1, 1, 200, 40], [900, 30, 0, 512], padded=(8, 256))
    lists = attention_tile_lists(facts, 4, kernels.PREFILL_TC_ROWS, 8, 0, 128, 148)
    assert lists.narrow_cap == 8 and lists.wide_cap >= max(16, len(lists.wide))
    assert lists.signature() == (lists.narrow_cap, lists.wide_cap, lists.shared)
    words = lists.words().reshape(-1, 4)
    assert words.shape[0] == lists.narrow_cap + lists.wide_cap
    assert [tuple(w) for w in words[:len(lists.narrow)]] == lists.narrow
    assert (words[len(lists.narrow):lists.narrow_cap] == 0).all()                           # entries without tokens
    assert [tuple(w) for w in words[lists.narrow_cap:lists.narrow_cap + len(lists.wide)]] == lists.wide
    only_wide = attention_tile_lists(facts_of([300], [0], padded=(1, 320)), 4, kernels.PREFILL_TC_ROWS, 8, 0, 128, 148)
    assert only_wide.narrow_cap == 0 and only_wide.wide_cap >= 16


def test_shares_of_the_keys_fit_the_gpu():
    """The split rule of the kernels for few rows: every share has two blocks of keys at least, all CTAs are
    resident at once, and clusters of 8 are not taken where they would need nearly all that the GPU holds."""
    from mini_rsglang_b200.parts.attention import choose_splits
    room = {2: 148, 4: 71, 8: 33, 16: 14}.get          # what a B200 states for the decode attention at heads of 128
    sms = 148
    for context in (64, 200, 1024, 4096, 8192, 16384, 65536):
        for tiles in (1, 2, 3, 4, 6, 8, 16, 32, 64, 128):
            for nkv in (1, 2, 8):
                plain = choose_splits(tiles, nkv, context, sms)
                fitted = choose_splits(tiles, nkv, context, sms, clusters=room)
                for splits in (plain, fitted):
                    assert 1 <= splits <= 64
                    assert splits == 1 or splits * 2 <= max(2, -(-context // 64))
                    assert splits == 1 or tiles * nkv * splits <= 2 * sms
                assert fitted in (plain, plain - 1)
                if fitted != plain:
                    assert plain in (8, 16) and tiles * nkv * 5 > room(plain) * 4
    assert choose_splits(4, 8, 8192, sms) == 8 and choose_splits(4, 8, 8192, sms, clusters=room) == 7
    assert choose_splits(2, 8, 8192, sms, clusters=room) == 8           # 16 clusters of 33: they fit
    assert choose_splits(1, 8, 16384, sms, clusters=room) == 16
    assert choose_splits(1, 8, 32768, sms, clusters=room) == 32         # more than a cluster has: they meet through memory
    assert choose_splits(2, 8, 32768, sms, clusters=room) == 15         # 16 clusters of 16 do not fit


def test_one_round_of_entries_pairs_early_tiles_with_late_ones():
    """With one round of CTAs (more than half the SMs, not more than all) the tiles of a portion are paired first with
    last: every entry then walks about as many blocks of keys as any other."""
    tokens = 1024
    facts = facts_of([tokens], [0])
    lists = attention_tile_lists(facts, 4, kernels.PREFILL_TC_ROWS, 8, 0, 128, 148)
    per_tile = kernels.PREFILL_TC_ROWS // 2 // 4
    assert len(lists.wide) == tokens // per_tile // 2 and not lists.shared and not lists.narrow
    work = []
    for seq, first, count, share in lists.wide:
        gap = share >> 16
        assert share & 0xFFFF == 0 and count == 2 * per_tile
        a, b = first // per_tile, (first + per_tile + gap) // per_tile
        assert a + b == tokens // per_tile - 1                     # first with last, second with last but one, ...
        work.append(-(-(a + 1) * per_tile // 128) + -(-(b + 1) * per_tile // 128))
    assert max(work) - min(work) <= 1

    def gaps(lengths, starts, window=0):
        return [share >> 16 for _, _, _, share in attention_tile_lists(facts_of(lengths, starts), 4, kernels.PREFILL_TC_ROWS, 8, window, 128, 148).wide]
    assert not any(gaps([2048], [0]))               # more CTAs than SMs: the rounds balance themselves
    assert not any(gaps([1024], [0], window=256))   # with a window every tile walks the same few blocks
    assert not any(gaps([256], [4096]))             # few CTAs: shares of the keys instead
