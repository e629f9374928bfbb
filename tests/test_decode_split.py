"""The key-range split of decode attention (a pure function of the longest context, the rows and the
kv heads): ranges of whole pages and whole rounds of the kernel's four warps, no more CTAs than one
wave of the kernel, halves beyond a wave, and one choice for a whole bucket of 1024 contexts."""
import pytest

from fellm_b200 import ops


@pytest.mark.parametrize("max_len", [1, 63, 64, 100, 900, 1024, 1025, 2049, 4000, 8192, 70000])
@pytest.mark.parametrize("rows,kv_heads", [(1, 1), (1, 8), (4, 2), (8, 8), (16, 8), (32, 8), (64, 8), (200, 4)])
def test_split_properties(max_len, rows, kv_heads):
    split_len, max_splits = ops.decode_split(max_len, rows, kv_heads)
    bucket = -(-max_len // 1024) * 1024
    assert split_len % 64 == 0 and split_len >= 64
    if split_len > 256:
        assert split_len % 256 == 0                       # whole rounds of four warps, a page each
    assert max_splits >= 1 and max_splits * split_len >= bucket >= max_len
    assert (max_splits - 1) * split_len < bucket          # no range without a key of the bucket
    items = rows * kv_heads
    if items <= ops.decode_target_ctas():
        assert items * max_splits <= max(ops.decode_target_ctas(), items)      # one wave
    elif bucket >= 128:
        assert max_splits == 2                            # more than a wave even unsplit: halves


def test_one_choice_for_a_bucket_of_contexts():
    """A decode step's CUDA graph holds the split: it must not change while contexts grow inside a bucket."""
    for rows, kv in [(1, 8), (8, 8), (64, 8)]:
        for lo in (1, 1025, 2049, 7169):
            choices = {ops.decode_split(n, rows, kv) for n in range(lo, lo + 1023, 37)}
            assert len(choices) == 1, (rows, kv, lo, choices)


def test_bench_shape():
    assert ops.decode_split(2049, 8, 8) == (512, 6)       # batch 8, 8 kv heads: 6 ranges of 8 pages for up to 3072 keys


def test_scratch_sized_once_covers_every_step_an_engine_can_run():
    """An engine reserves the split kernel's scratch before its first step, so that no captured
    graph outlives a buffer: the size must cover every row count and every context bucket."""
    import random
    for max_rows, H, G, hd, n_ctx in [(8, 4, 2, 16, 512), (64, 16, 8, 64, 8192), (200, 32, 4, 128, 5000), (3, 6, 1, 48, 1024)]:
        floats, counters = ops.decode_scratch_need(max_rows, H, G, hd, n_ctx)
        rng = random.Random(max_rows)
        for _ in range(300):
            rows, max_len = rng.randrange(1, max_rows + 1), rng.randrange(1, n_ctx + 1)
            _, max_splits = ops.decode_split(max_len, rows, G)
            assert rows * H * max_splits * (hd + 2) <= floats and rows * G <= counters
