"""The host rule that shares a sequence's keys among blocks in decode attention (no device
needed): the split count with the least estimated time, never more than there is work, never above 32
(what the merge kernel fetches in one round)."""
from torchless_rs_b200.csrc.attention_bf16 import TARGET_BLOCKS, decode_splits


def test_the_measured_choices_at_mistral_7b_sizes():
    # 8 kv heads, context 4096: the split counts that the timings of the decode kernel were taken at
    assert decode_splits(1, 8, 4096, None) == 32
    assert decode_splits(8, 8, 4096, None) == 4
    assert decode_splits(16, 8, 4096, None) == 2
    assert decode_splits(32, 8, 4096, None) == 1
    assert decode_splits(64, 8, 4096, None) == 1


def test_more_pairs_than_one_wave_are_cut_finer():
    # measured: 20 sequences 57 us in 3 splits against 63 us in 1; 40 sequences 111 us in 4 against 138 us in 1;
    # 48 sequences 123 us in 2 or 3 against 142 us in 1; 24 and 28 sequences are best left whole
    assert decode_splits(20, 8, 4096, None) == 3
    assert decode_splits(40, 8, 4096, None) in (3, 4)
    assert decode_splits(48, 8, 4096, None) in (2, 3)
    assert decode_splits(24, 8, 4096, None) == 1
    assert decode_splits(28, 8, 4096, None) == 1


def test_short_contexts_are_not_split_for_nothing():
    # 256 tokens: a merge kernel costs more than the split saves (8 sequences: 5.4 us whole, 6.3 us in 3 splits)
    assert decode_splits(8, 8, 256, None) == 1
    assert decode_splits(8, 8, 1024, None) == 4
    assert decode_splits(1, 8, 1024, None) in (8, 9)


def test_bounds():
    for nkv in (1, 2, 8):
        for hd in (64, 128):
            for length in (1, 31, 100, 4096, 32768, 1 << 20):
                for batch in (1, 2, 4, 8, 16, 20, 40, 64, 1024):
                    s = decode_splits(batch, nkv, length, None, TARGET_BLOCKS, hd)
                    assert 1 <= s <= 32
                    assert s <= (length + 31) // 32 + 1                   # never more splits than 32-key groups
                    assert s <= 4 or batch * nkv * s <= TARGET_BLOCKS     # many splits only within one wave


def test_a_window_bounds_the_work():
    assert decode_splits(1, 8, 32768, 1024) == decode_splits(1, 8, 1024, None)
    assert decode_splits(1, 8, 100, 4096) == decode_splits(1, 8, 100, None)
