"""The engine against the plain implementation, under every way of cutting the
work: whole prompts, the last 32 tokens one by one, batches of unequal lengths whose
shorter requests end earlier, one batch after another so that slots are used again."""
import numpy as np
import pytest

from helpers_gpu import TinyModel, assert_close
from tiny import random_tokens

pytestmark = pytest.mark.gpu

DTYPES = ["float32", "bfloat16"]
NAMES = ["A", "B", "C", "D", "E"]


@pytest.fixture(scope="module", params=[(n, d) for n in NAMES for d in DTYPES],
                ids=lambda p: f"{p[0]}-{p[1]}")
def tiny(request):
    name, dtype = request.param
    return TinyModel(name, dtype, seed=11 + ord(name), max_tokens=1024)


def _requests(tiny, lengths, seed):
    rng = np.random.default_rng(seed)
    return [random_tokens(rng, n, tiny.cfg["vocab_size"]) for n in lengths]


def test_whole_alone(tiny):
    for toks in _requests(tiny, [1, 5, 23, 70, 150], 1):
        (s,) = tiny.engine.start_sequences(1)
        got = tiny.step_np([s], [toks], "all")
        tiny.engine.end_sequences([s])
        assert_close(got, tiny.reference(toks), tiny.dtype, f"whole n={len(toks)}")
    tiny.engine.cache.check()


def test_last_32_one_by_one(tiny):
    for toks in _requests(tiny, [33, 50, 97, 140], 2):
        ref = tiny.reference(toks)
        n = len(toks)
        (s,) = tiny.engine.start_sequences(1)
        head = n - 32
        got = [tiny.step_np([s], [toks[:head]], "all")]
        for i in range(head, n):
            got.append(tiny.step_np([s], [[toks[i]]], "last"))
        tiny.engine.end_sequences([s])
        assert_close(np.concatenate(got), ref, tiny.dtype, f"last32 n={n}")
    tiny.engine.cache.check()


def test_first_tokens_decoded_from_scratch(tiny):
    """A sequence that starts with a one-token prompt and goes on token by token."""
    (toks,) = _requests(tiny, [40], 3)
    (s,) = tiny.engine.start_sequences(1)
    got = [tiny.step_np([s], [[t]], "last") for t in toks]
    tiny.engine.end_sequences([s])
    assert_close(np.concatenate(got), tiny.reference(toks), tiny.dtype, "from scratch")


def test_unequal_batches_slots_used_again(tiny):
    """Three batches one after another in a cache that holds only one batch at a
    time; in each, prompts of unequal lengths start together, then every request
    goes on one token per step until its tokens run out."""
    lens = [[5, 11, 23], [1, 19], [64, 65, 3, 30]]
    prefix = [[3, 5, 20], [1, 7], [60, 33, 2, 17]]
    seen_slots = []
    for b, (ls, ps) in enumerate(zip(lens, prefix)):
        reqs = _requests(tiny, ls, 10 + b)
        slots = tiny.engine.start_sequences(len(reqs))
        seen_slots.append(tuple(slots))
        got = [[] for _ in reqs]
        out = tiny.step_np(slots, [r[:p] for r, p in zip(reqs, ps)], "all")
        o = 0
        for i, p in enumerate(ps):
            got[i].append(out[o:o + p]); o += p
        fed = list(ps)
        live = list(range(len(reqs)))
        while True:
            done = [i for i in live if fed[i] >= len(reqs[i])]
            if done:
                tiny.engine.end_sequences([slots[i] for i in done])
                live = [i for i in live if i not in done]
            if not live:
                break
            out = tiny.step_np([slots[i] for i in live], [[reqs[i][fed[i]]] for i in live], "last")
            for j, i in enumerate(live):
                got[i].append(out[j:j + 1]); fed[i] += 1
        for i, r in enumerate(reqs):
            assert_close(np.concatenate(got[i]), tiny.reference(r), tiny.dtype,
                         f"batch {b} request {i} (n={len(r)})")
        tiny.engine.cache.check()
    assert seen_slots[0][0] == seen_slots[1][0] == seen_slots[2][0], "slots are not used again"
    assert tiny.engine.cache.slots.held_count == 0
    for g in tiny.engine.cache.paged:
        assert g.pool.held_count == 0


def test_long_decode(tiny):
    """200 decoded tokens after a short prompt: crosses page borders and, with a
    window, frees pages on the way."""
    (toks,) = _requests(tiny, [210], 5)
    ref = tiny.reference(toks)
    (s,) = tiny.engine.start_sequences(1)
    got = [tiny.step_np([s], [toks[:10]], "all")]
    for t in toks[10:]:
        got.append(tiny.step_np([s], [[t]], "last"))
    tiny.engine.cache.check()
    tiny.engine.end_sequences([s])
    assert_close(np.concatenate(got), ref, tiny.dtype, "long decode")
