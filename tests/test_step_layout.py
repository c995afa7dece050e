"""The host library's layout of a step (`csrc/host/step_batch.cc`) and the bound by which the step
function sizes its buffers: a padded step of single decoded tokens needs the same words however many
of its sequences are real, so a recorded step's fixed buffers never fall short."""
import ctypes

import numpy as np
import pytest

from mini_rsglang_b200.cache.manager import CacheGroup, CacheManager, host_api
from mini_rsglang_b200.engine.runner import step_layout_bound


def build(cache, sequences, pad_to, width, max_seq_len, cap):
    """Calls `mrs_step_build` for single decoded tokens of `sequences` = [(request, position)]."""
    lib = host_api()
    fn = lib.mrs_step_build
    fn.restype = ctypes.c_int64
    fn.argtypes = [ctypes.c_void_p, ctypes.c_int] + [ctypes.c_void_p] * 6 + [
        ctypes.c_int, ctypes.c_int, ctypes.c_int64, ctypes.c_int64, ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p]
    n = len(sequences)
    requests = np.array([r for r, _ in sequences], dtype=np.int64)
    starts = np.array([p for _, p in sequences], dtype=np.int64)
    counts = np.ones(n, dtype=np.int32)
    tokens = np.zeros(n, dtype=np.int32)
    want_counts = np.ones(n, dtype=np.int32)
    want = np.zeros(n, dtype=np.int32)
    layout = np.zeros(17, dtype=np.int64)
    buf = np.zeros(cap, dtype=np.int32)
    used = fn(cache.handle, n, requests.ctypes.data, starts.ctypes.data, counts.ctypes.data, tokens.ctypes.data,
              want_counts.ctypes.data, want.ctypes.data, pad_to, width, max_seq_len, 1000, buf.ctypes.data, cap,
              layout.ctypes.data)
    return int(used), layout, buf


@pytest.mark.parametrize("max_seq_len,bucket", [(768, 128), (768, 64), (256, 128), (1792, 32), (752, 256)])
def test_a_padded_step_needs_the_same_words_however_many_sequences_are_real(max_seq_len, bucket):
    page = 16
    width = -(-max_seq_len // page)
    cache = CacheManager([CacheGroup("full", 0, 4 * bucket)], page, bucket)
    for r in range(bucket):
        cache.open(r + 1)
        cache.extend(r + 1, 3)
    bound = step_layout_bound(bucket, bucket, width, 1)
    few, many = bucket // 2 + 1, bucket
    used_few, layout_few, _ = build(cache, [(r + 1, 2) for r in range(few)], bucket, width, max_seq_len, bound)
    used_many, layout_many, _ = build(cache, [(r + 1, 2) for r in range(many)], bucket, width, max_seq_len, bound)
    assert used_few == used_many > 0
    assert used_many <= bound
    assert list(layout_few[:12]) == list(layout_many[:12])        # the same offsets: a recording's tensors stay put
    # the buffers of a recording are sized by the bound of its first step, rounded up to a power of two: what a
    # later step with more real sequences needs is never more
    size_at_recording = max(4096, 1 << (step_layout_bound(bucket, bucket, width, 1) - 1).bit_length())
    assert used_many <= size_at_recording


def test_the_bound_covers_mixed_steps_and_too_small_a_buffer_is_reported():
    page = 4
    cache = CacheManager([CacheGroup("full", 0, 64), CacheGroup("window", 8, 64)], page, 4)
    lib = host_api()
    fn = lib.mrs_step_build
    fn.restype = ctypes.c_int64
    fn.argtypes = [ctypes.c_void_p, ctypes.c_int] + [ctypes.c_void_p] * 6 + [
        ctypes.c_int, ctypes.c_int, ctypes.c_int64, ctypes.c_int64, ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p]
    counts = np.array([7, 1, 13], dtype=np.int32)
    for r, n in enumerate(counts):
        cache.open(r + 1)
        cache.extend(r + 1, int(n))
    requests = np.array([1, 2, 3], dtype=np.int64)
    starts = np.zeros(3, dtype=np.int64)
    tokens = np.arange(int(counts.sum()), dtype=np.int32)
    want_counts = np.array([2, 1, 0], dtype=np.int32)
    want = np.array([0, 6, 0], dtype=np.int32)
    layout = np.zeros(14 + 3 * 2, dtype=np.int64)
    bound = step_layout_bound(int(counts.sum()), 3, -(-64 // page), 2)
    buf = np.zeros(bound, dtype=np.int32)
    used = fn(cache.handle, 3, requests.ctypes.data, starts.ctypes.data, counts.ctypes.data, tokens.ctypes.data,
              want_counts.ctypes.data, want.ctypes.data, 0, 0, 64, 1000, buf.ctypes.data, bound, layout.ctypes.data)
    assert 0 < used <= bound
    assert list(layout[:4]) == [21, 3, 3, 0]
    assert list(buf[layout[10]:layout[10] + 3]) == [0, 6, 7]           # wanted rows in the flat batch
    small = fn(cache.handle, 3, requests.ctypes.data, starts.ctypes.data, counts.ctypes.data, tokens.ctypes.data,
               want_counts.ctypes.data, want.ctypes.data, 0, 0, 64, 1000, buf.ctypes.data, 16, layout.ctypes.data)
    assert small == -7 and layout[0] == used


def test_a_step_padded_to_fixed_shapes_keeps_its_layout_and_its_added_rows_write_nothing():
    """A mixed step padded to fixed rows and sequences: the layout depends on the padded sizes alone, the added
    sequences have no rows, the added rows write nothing, and the wanted rows are the real ones, then row 0."""
    page, width = 4, 16
    cache = CacheManager([CacheGroup("full", 0, 64)], page, 8)
    lib = host_api()
    fn = lib.mrs_step_build_padded
    fn.restype = ctypes.c_int64
    fn.argtypes = [ctypes.c_void_p, ctypes.c_int] + [ctypes.c_void_p] * 6 + [
        ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int64, ctypes.c_int64, ctypes.c_void_p, ctypes.c_int64,
        ctypes.c_void_p]

    def build(counts, want_counts, want, pad_to, pad_rows):
        n = len(counts)
        counts = np.array(counts, dtype=np.int32)
        requests = np.arange(1, n + 1, dtype=np.int64)
        starts = np.zeros(n, dtype=np.int64)
        tokens = np.arange(1, int(counts.sum()) + 1, dtype=np.int32)
        want_counts = np.array(want_counts, dtype=np.int32)
        want = np.array(want, dtype=np.int32)
        layout = np.zeros(17, dtype=np.int64)
        bound = step_layout_bound(pad_rows, pad_to, width, 1)
        buf = np.full(bound, 77, dtype=np.int32)
        used = fn(cache.handle, n, requests.ctypes.data, starts.ctypes.data, counts.ctypes.data, tokens.ctypes.data,
                  want_counts.ctypes.data, want.ctypes.data, pad_to, pad_rows, width, 64, 1000, buf.ctypes.data, bound,
                  layout.ctypes.data)
        return int(used), layout, buf

    for r, n in enumerate((7, 1, 13)):
        cache.open(r + 1)
        cache.extend(r + 1, n)
    used, layout, buf = build([7, 1, 13], [0, 1, 1], [0, 12], 4, 32)
    assert used > 0, lib.mrs_step_last_error()
    T, B, R, decode = (int(v) for v in layout[:4])
    assert (T, B, R, decode) == (32, 4, 4, 0)
    assert list(buf[layout[7]:layout[7] + 5]) == [0, 7, 8, 21, 21]              # the added sequence has no rows
    assert list(buf[layout[10]:layout[10] + 4]) == [7, 20, 0, 0]                # real wanted rows, then row 0
    slots = buf[layout[14]:layout[14] + T]
    assert (slots[:21] >= 0).all() and (slots[21:] == -1).all()                 # added rows write nothing
    assert (buf[layout[6] + 21:layout[6] + T] == B - 1).all() and (buf[layout[5] + 21:layout[5] + T] == 0).all()
    assert (buf[layout[12] + 3 * width:layout[12] + 4 * width] == 0).all()      # the added sequence reads page 0
    # another step of the same padded sizes: the same offsets and the same need
    used2, layout2, _ = build([2, 1], [1, 1], [1, 0], 4, 32)
    assert used2 == used and list(layout2[:12]) == list(layout[:12])
    # refusals: two wanted places in a sequence, fewer rows than the step has
    assert build([7, 1], [2, 0], [0, 1], 4, 32)[0] == -6
    assert build([7, 1, 13], [0, 0, 0], [], 4, 16)[0] == -6
