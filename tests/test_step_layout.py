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
