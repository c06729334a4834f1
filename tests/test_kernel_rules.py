"""Host-side rules of the kernels' wrappers that need no device: how a decode step's keys are
cut for the split-key attention (vipera.rs_b200/kernels/ops.py, decode_splits).  A cut that does
not cover the longest history would leave keys out without any error, so the properties are
checked over every size a step can have."""
import random

import vipera_rs_b200  # noqa: F401
from vipera_rs_b200.kernels import ops


def _check(entries, kv_heads, keys, sms):
    chunk, splits = ops.decode_splits(entries, kv_heads, keys, sms)
    assert chunk >= 128 and chunk % 128 == 0, (entries, kv_heads, keys, sms, chunk)
    assert 1 <= splits <= 64, (entries, kv_heads, keys, sms, splits)        # the combine kernel holds at most 128
    assert chunk * splits >= keys, (entries, kv_heads, keys, sms, chunk, splits)
    # splits past the longest history are allowed (their blocks leave at once), but never more
    # than the next power of two of keys would need
    assert chunk * (splits - 1) < 2 * max(keys, 128), (entries, kv_heads, keys, sms, chunk, splits)
    return chunk, splits


def test_the_cut_of_a_decode_steps_keys_covers_every_history():
    for keys in list(range(1, 700)) + [2047, 2048, 2049, 4096, 8191, 8192, 32768, 131072, 1000003]:
        for entries, kv_heads in ((1, 1), (1, 2), (8, 2), (64, 2), (48, 8), (256, 8), (1000, 1)):
            _check(entries, kv_heads, keys, 148)
    drawn = random.Random(20240611)
    for _ in range(5000):
        _check(drawn.randint(1, 512), drawn.choice([1, 2, 3, 4, 8, 16]), drawn.randint(1, 300000),
               drawn.choice([1, 8, 108, 132, 148, 160]))


def test_short_histories_of_few_entries_are_cut_into_tiles_of_128_keys():
    """Every block then asks for all its keys at once, before it waits for the kernel ahead."""
    for entries in (1, 2, 8):
        assert ops.decode_splits(entries, 2, 2048, 148) == (128, 16)
    assert ops.decode_splits(8, 2, 8192, 148) == (128, 64)
    assert ops.decode_splits(8, 2, 9216, 148) == (256, 64)     # as for 16,384 keys
    # many entries with long histories: fewer and longer splits, whole waves of three blocks an SM
    chunk, splits = ops.decode_splits(64, 2, 8192, 148)
    assert chunk > 128 and 64 * 2 * splits <= 2 * 3 * 148


def test_the_width_classes_of_decode_graphs_hold_the_table_and_little_more():
    """vipera.rs_b200/engine/runner.py, _width_bucket: a class is never narrower than the table,
    never shrinks as the table grows, and above 128 pages is at most an eighth of its octave
    wider than the table."""
    from vipera_rs_b200.engine.runner import _width_bucket

    before = 0
    for pages in range(1, 70000):
        width = _width_bucket(pages)
        assert width >= pages and width >= before
        if pages > 128:
            assert width - pages < max(16, pages // 8 + 1), (pages, width)
        before = width
    assert [_width_bucket(p) for p in (1, 8, 9, 128, 129, 133, 517, 2049)] == [8, 8, 16, 128, 144, 144, 576, 2304]
