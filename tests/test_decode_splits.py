"""The host rule that shares a sequence's keys among blocks in decode attention (no device
needed): enough blocks for one wave of the GPU, never more than there is work, never above 32 (what the merge kernel fetches in one round)."""
from torchless_rs_b200.csrc.attention_bf16 import TARGET_BLOCKS, decode_splits


def test_the_measured_choices_at_mistral_7b_sizes():
    # 8 kv heads, context 4096: the split counts that the timings of the decode kernel were taken at
    assert decode_splits(1, 8, 4096, None) == 32
    assert decode_splits(8, 8, 4096, None) == 4
    assert decode_splits(16, 8, 4096, None) == 2
    assert decode_splits(64, 8, 4096, None) == 1


def test_bounds_and_monotony():
    for nkv in (1, 2, 8):
        for length in (1, 31, 100, 4096, 32768, 1 << 20):
            last = None
            for batch in (1, 2, 4, 8, 16, 64, 1024):
                s = decode_splits(batch, nkv, length, None)
                assert 1 <= s <= 32
                assert s == 1 or batch * nkv * s <= TARGET_BLOCKS     # one wave of blocks at most
                assert s <= (length + 31) // 32 + 1                   # never more splits than 32-key groups
                assert last is None or s <= last                      # more sequences, fewer splits each
                last = s


def test_a_window_bounds_the_work():
    assert decode_splits(1, 8, 32768, 1024) == decode_splits(1, 8, 1024, None)
    assert decode_splits(1, 8, 100, 4096) == decode_splits(1, 8, 100, None)
