"""The host arithmetic of a step (no device needed): where the packed tokens of unequal
sequences lie, their positions after what the cache already holds, and the wanted rows."""
import numpy as np
import pytest

from torchless_rs_b200.engine.batch import layout_step


def test_prompts_of_unequal_lengths_are_packed_one_after_the_other():
    lay = layout_step(past_lens=[0, 0, 0], counts=[3, 1, 2], slots=[5, 0, 2],
                      tokens=[[7, 8, 9], [4], [1, 2]], want=[[0, 2], [], [1]])
    assert lay["tokens"].tolist() == [7, 8, 9, 4, 1, 2]
    assert lay["token_seq"].tolist() == [0, 0, 0, 1, 2, 2]
    assert lay["token_pos"].tolist() == [0, 1, 2, 0, 0, 1]
    assert lay["seq_start"].tolist() == [0, 3, 4, 6]
    assert lay["seq_len"].tolist() == [3, 1, 2]
    assert lay["seq_slot"].tolist() == [5, 0, 2]
    assert lay["want_rows"].tolist() == [0, 2, 5]          # order of the entries, then of `want`
    assert lay["token_from"].tolist() == [-1] * 6
    assert all(a.dtype == np.int32 for a in lay.values())


def test_a_decode_step_continues_at_each_sequence_s_own_length():
    lay = layout_step(past_lens=[3, 70, 64], counts=[1, 1, 1], slots=[1, 2, 3],
                      tokens=[[11], [12], [13]], want=[[0], [0], [0]])
    assert lay["token_pos"].tolist() == [3, 70, 64]
    assert lay["seq_len"].tolist() == [4, 71, 65]
    assert lay["want_rows"].tolist() == [0, 1, 2]


def test_a_chunk_after_a_prefix_and_nothing_wanted():
    lay = layout_step(past_lens=[10], counts=[4], slots=[0], tokens=[[1, 2, 3, 4]], want=[[]])
    assert lay["token_pos"].tolist() == [10, 11, 12, 13]
    assert lay["want_rows"].size == 0


def test_a_wanted_place_outside_the_entry_is_refused():
    with pytest.raises(ValueError, match="outside the 2 tokens of entry 1"):
        layout_step([0, 0], [1, 2], [0, 1], [[1], [2, 3]], [[0], [2]])
    with pytest.raises(ValueError):
        layout_step([0], [1], [0], [[1]], [[-1]])
