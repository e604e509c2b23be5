"""The cache's host side: slots and pages are never lost, held twice or freed twice;
windows give pages back; capacity errors change nothing (no device needed)."""
import numpy as np
import pytest
import torch

from torchless_rs_b200.cache import (PAGE, Cache, CacheCapacityError, CacheRollbackError, CacheStateError, FreeList,
                                     PagedKVRequest, StateRequest)


def _cache(max_tokens=1024, window=None, max_slots=None, extra=()):
    reqs = [PagedKVRequest(2, 16, window), PagedKVRequest(2, 16, window)] + list(extra)
    return Cache(reqs, max_tokens, max_slots, None, torch.float32, "cpu")


def test_free_list_states():
    f = FreeList(4, "thing")
    a = f.take(3)
    assert a == [0, 1, 2] and f.free_count == 1
    with pytest.raises(CacheCapacityError):
        f.take(2)
    f.give_back([1])
    with pytest.raises(CacheStateError, match="not held"):
        f.give_back([1])
    with pytest.raises(CacheStateError, match="does not exist"):
        f.give_back([7])
    assert f.take(2) == [1, 3]      # lowest first: reuse is deterministic
    f.check()


def test_slots_and_pages_come_back_and_are_used_again():
    c = _cache()
    s = c.acquire(3)
    c.prepare(s, [5, 64, 65])
    c.commit(s, [5, 64, 65])
    g = c.paged[0]
    assert g.pool.held_count == 1 + 1 + 2 and c.lengths[s[2]] == 65
    c.check()
    c.release([s[1]])
    assert g.pool.held_count == 3
    with pytest.raises(CacheStateError, match="not held"):
        c.release([s[1]])
    with pytest.raises(CacheStateError, match="not held"):
        c.prepare([s[1]], [3])
    (again,) = c.acquire(1)
    assert again == s[1] and c.length(again) == 0
    c.prepare([again], [200])
    c.commit([again], [200])
    c.check()
    c.release([s[0], s[2], again])
    assert g.pool.held_count == 0 and c.slots.held_count == 0
    c.check()


def test_same_slot_twice_in_a_step_is_refused():
    c = _cache()
    (s,) = c.acquire(1)
    with pytest.raises(CacheStateError, match="twice"):
        c.prepare([s, s], [3, 3])


def test_full_cache_raises_and_changes_nothing():
    c = _cache(max_tokens=4 * PAGE)
    s = c.acquire(2)
    c.prepare(s, [PAGE, 2 * PAGE])
    c.commit(s, [PAGE, 2 * PAGE])
    before = (c.paged[0].table_host.copy(), c.paged[0].pool.free_count)
    with pytest.raises(CacheCapacityError, match="full"):
        c.prepare(s, [2 * PAGE, 3 * PAGE])       # needs two more pages, one is free
    assert np.array_equal(before[0], c.paged[0].table_host) and before[1] == c.paged[0].pool.free_count
    with pytest.raises(CacheCapacityError, match="longer"):
        c.prepare([s[0]], [5 * PAGE])
    c.check()


def test_window_gives_pages_back_while_decoding():
    w = 100
    c = _cache(max_tokens=4096, window=w)
    (s,) = c.acquire(1)
    g = c.paged[0]
    c.prepare([s], [300])            # a prompt longer than the window: all pages for the step
    assert g.pool.held_count == 5
    c.commit([s], [300])             # next position 300 sees keys 201..: pages 0-2 go back
    assert g.first_live[s] == 3 and g.pool.held_count == 2
    for n in range(301, 700):
        c.prepare([s], [n])
        c.commit([s], [n])
        first_needed = n - w + 1
        assert g.first_live[s] == first_needed // PAGE
        assert g.pool.held_count <= (w + PAGE - 1) // PAGE + 1
        c.check()
    assert all(int(p) == -1 for p in g.table_host[s, :g.first_live[s]])
    c.release([s])
    assert g.pool.held_count == 0


def test_groups_by_need_and_state_is_zeroed_on_acquire():
    reqs = [PagedKVRequest(2, 16, None), PagedKVRequest(2, 16, 32), PagedKVRequest(2, 16, None),
            StateRequest((3, 4)), None]
    c = Cache(reqs, 512, 4, None, torch.float32, "cpu")
    assert len(c.paged) == 2 and len(c.states) == 1
    assert c.view(0).group is c.view(2).group and c.view(0).group is not c.view(1).group
    assert c.view(4) is None
    assert c.view(0).k_pages.shape == (8, 2, PAGE, 16) and c.view(0).v_pages.shape == (8, 2, 16, PAGE)
    st = c.view(3)
    assert st.shape == (4, 3, 4)
    (s,) = c.acquire(1)
    st[s] += 7.0
    c.release([s])
    (s2,) = c.acquire(1)
    assert s2 == s and float(c.view(3)[s2].abs().sum()) == 0.0


def test_max_tokens_rounds_up_to_pages():
    c = _cache(max_tokens=130)
    assert c.max_tokens == 192 and c.paged[0].n_pages == 3


def test_truncate_gives_whole_pages_back_and_reset_empties_the_slot():
    c = _cache()
    s, other = c.acquire(2)
    c.prepare([s, other], [300, 10])
    c.commit([s, other], [300, 10])
    g = c.paged[0]
    assert g.pool.held_count == 5 + 1
    c.truncate(s, 300)                      # nothing to do
    c.truncate(s, 129)                      # pages 0-2 stay (129 tokens need three)
    assert c.length(s) == 129 and g.n_cols[s] == 3 and g.pool.held_count == 3 + 1
    assert all(int(p) == -1 for p in g.table_host[s, 3:])
    c.check()
    c.prepare([s], [200])                   # goes on from 129
    c.commit([s], [200])
    assert g.pool.held_count == 4 + 1
    with pytest.raises(ValueError):
        c.truncate(s, 201)
    with pytest.raises(ValueError):
        c.truncate(s, -1)
    c.reset(s)
    assert c.length(s) == 0 and g.n_cols[s] == 0 and g.pool.held_count == 1 and c.slots.is_held(s)
    c.check()
    c.release([s, other])
    with pytest.raises(CacheStateError, match="not held"):
        c.truncate(s, 0)
    assert g.pool.held_count == 0
    c.check()


def test_truncate_refuses_what_a_window_has_given_back():
    w = 100
    c = _cache(max_tokens=4096, window=w)
    (s,) = c.acquire(1)
    g = c.paged[0]
    c.prepare([s], [300])
    c.commit([s], [300])                    # keys before 192 are gone (pages 0-2)
    assert g.first_live[s] == 3
    before = (g.table_host.copy(), g.pool.free_count, c.length(s))
    with pytest.raises(CacheRollbackError, match="window"):
        c.truncate(s, 290)                  # position 290 sees keys from 191 on: page 2 is gone
    assert np.array_equal(before[0], g.table_host) and before[1] == g.pool.free_count and c.length(s) == before[2]
    c.truncate(s, 291)                      # sees keys from 192 on: possible
    assert c.length(s) == 291 and g.pool.held_count == 2
    c.check()
    c.reset(s)                              # always possible
    assert g.first_live[s] == 0 and g.pool.held_count == 0
    c.prepare([s], [70])
    c.commit([s], [70])
    c.check()


def test_truncate_with_state_of_fixed_size_only_resets():
    reqs = [PagedKVRequest(2, 16, None), StateRequest((3,))]
    c = Cache(reqs, 512, 4, None, torch.float32, "cpu")
    (s,) = c.acquire(1)
    c.prepare([s], [80])
    c.commit([s], [80])
    c.view(1)[s] += 2.0
    with pytest.raises(CacheRollbackError, match="state"):
        c.truncate(s, 40)
    assert c.length(s) == 80
    c.reset(s)
    assert c.length(s) == 0 and float(c.view(1)[s].abs().sum()) == 0.0 and c.paged[0].pool.held_count == 0
    c.check()
