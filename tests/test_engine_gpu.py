"""The engine against the plain implementation, under every way of cutting the
work: whole prompts, the last 32 tokens one by one, batches of unequal lengths whose
shorter requests end earlier, one batch after another so that slots are used again."""
import numpy as np
import pytest

from helpers_gpu import TinyModel, assert_close
from tiny import random_tokens

pytestmark = pytest.mark.gpu

DTYPES = ["float32", "bfloat16"]
NAMES = ["A", "B", "C", "D", "E", "F"]


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


def test_mixed_step_decode_rows_fresh_prompt_and_chunk(tiny):
    """One step that holds a sequence going on by one token, a sequence going on by a chunk
    of 130 tokens (on a slot that already holds 20) and a sequence that starts."""
    x, y, z = _requests(tiny, [72, 151, 38], 21)
    sx, sy, sz = tiny.engine.start_sequences(3)
    got = {0: [], 1: [], 2: []}
    out = tiny.step_np([sx, sy], [x[:70], y[:20]], "all")
    got[0].append(out[:70]); got[1].append(out[70:])
    out = tiny.step_np([sx, sy, sz], [[x[70]], y[20:150], z[:37]], "all")
    got[0].append(out[:1]); got[1].append(out[1:131]); got[2].append(out[131:])
    out = tiny.step_np([sz, sx, sy], [[z[37]], [x[71]], [y[150]]], "last")   # another row order
    got[2].append(out[0:1]); got[0].append(out[1:2]); got[1].append(out[2:3])
    tiny.engine.cache.check()
    tiny.engine.end_sequences([sx, sy, sz])
    for i, r in enumerate((x, y, z)):
        assert_close(np.concatenate(got[i]), tiny.reference(r), tiny.dtype, f"mixed step, request {i}")


def test_prompt_in_chunks_on_a_slot_that_holds_tokens(tiny):
    """A prompt of 300 tokens fed as 70 + 200 + 30: the second chunk brings more than 128 new
    tokens to a slot that is not empty (with a window, pages have been given back by then)."""
    (toks,) = _requests(tiny, [300], 22)
    (s,) = tiny.engine.start_sequences(1)
    got = [tiny.step_np([s], [toks[a:b]], "all") for a, b in ((0, 70), (70, 270), (270, 300))]
    tiny.engine.cache.check()
    tiny.engine.end_sequences([s])
    assert_close(np.concatenate(got), tiny.reference(toks), tiny.dtype, "prompt in chunks")


def test_prefill_in_several_steps_gives_each_prompts_last_logits(tiny):
    """`Engine.prefill` with a small number of tokens per step: four prompts of unequal lengths go
    in steps of 128 tokens each, the shorter ones run out earlier, and every prompt's last logits
    are those of the plain implementation; then the sequences decode one token together."""
    reqs = _requests(tiny, [300, 129, 40, 256], 41)
    slots = tiny.engine.start_sequences(4)
    staged = tiny.engine.stager.staged
    got = tiny.engine.prefill(slots, reqs, tokens_per_step=256).cpu().numpy().copy()
    # 128 + 128 + 44, 129 at once (one token gets no step of its own), 40, 128 + 128
    assert tiny.engine.stager.staged - staged == 3
    tiny.engine.cache.check()
    for i, r in enumerate(reqs):
        assert_close(got[i:i + 1], tiny.reference(r)[-1:], tiny.dtype, f"prefill in steps, prompt {i}")
    nxt = [int(g.argmax()) for g in got]
    dec = tiny.step_np(slots, [[t] for t in nxt], "last")
    tiny.engine.end_sequences(slots)
    for i, r in enumerate(reqs):
        assert_close(dec[i:i + 1], tiny.reference(list(r) + [nxt[i]])[-1:], tiny.dtype, f"decode after, {i}")
    # under the limit it is one step, and the same numbers
    slots = tiny.engine.start_sequences(4)
    one = tiny.engine.prefill(slots, reqs, tokens_per_step=4096).cpu().numpy().copy()
    tiny.engine.end_sequences(slots)
    assert_close(one, got, tiny.dtype, "one step against several")


def test_decode_across_a_length_bucket(tiny):
    """Decoding from 250 to 520 tokens: the recorded graph's key and the split of the keys
    among blocks change at 256 and at 512."""
    (toks,) = _requests(tiny, [520], 23)
    ref = tiny.reference(toks)
    (s,) = tiny.engine.start_sequences(1)
    got = [tiny.step_np([s], [toks[:250]], "all")]
    for t in toks[250:]:
        got.append(tiny.step_np([s], [[t]], "last"))
    tiny.engine.cache.check()
    tiny.engine.end_sequences([s])
    assert_close(np.concatenate(got), ref, tiny.dtype, "decode 250 -> 520")


def test_float16_folder_is_widened_exactly_on_the_32_bit_path():
    """A folder stored in float16, run in 32-bit: the engine computes with the stored values
    (11 bits of mantissa), not with their bfloat16 roundings, which would miss the 32-bit
    tolerance by an order of magnitude."""
    import torch
    tiny = TinyModel("B", "float32", seed=41, store=torch.float16)
    assert any(v.dtype == np.float32 and np.any(v != v.astype(np.float32).view(np.uint32).__and__(0xFFFF0000).view(np.float32))
               for v in tiny.weights.values()), "the stored values all fit bfloat16: the test shows nothing"
    (toks,) = _requests(tiny, [60], 42)
    (s,) = tiny.engine.start_sequences(1)
    got = [tiny.step_np([s], [toks[:50]], "all")] + [tiny.step_np([s], [[t]], "last") for t in toks[50:]]
    tiny.engine.end_sequences([s])
    assert_close(np.concatenate(got), tiny.reference(toks), "float32", "float16 folder in 32-bit")


def test_truncate_then_decode_again_gives_the_same_logits(tiny):
    """20 tokens decoded after a prompt, the sequence rolled back to the prompt, the same 20
    tokens decoded again: the same logits bit for bit; then rolled back to one token before
    the prompt's end and the prompt's last token fed alone."""
    (toks,) = _requests(tiny, [50], 31)
    ref = tiny.reference(toks)
    (s,) = tiny.engine.start_sequences(1)
    tiny.step_np([s], [toks[:30]], "last")
    first = [tiny.step_np([s], [[t]], "last") for t in toks[30:]]
    tiny.engine.truncate(s, 30)
    assert tiny.engine.length(s) == 30
    tiny.engine.cache.check()
    again = [tiny.step_np([s], [[t]], "last") for t in toks[30:]]
    assert all(np.array_equal(a, b) for a, b in zip(first, again)), "rolled back and run again: other logits"
    assert_close(np.concatenate(again), ref[30:], tiny.dtype, "after truncate")
    tiny.engine.truncate(s, 29)
    assert_close(tiny.step_np([s], [[toks[29]]], "last"), ref[29:30], tiny.dtype, "prompt's last token alone")
    tiny.engine.reset(s)
    assert tiny.engine.length(s) == 0
    assert_close(tiny.step_np([s], [toks[:9]], "all"), ref[:9], tiny.dtype, "after reset")
    tiny.engine.cache.check()
    tiny.engine.end_sequences([s])


def test_steady_decode_steps_advance_their_state_on_the_device(tiny):
    """Two sequences that go on token by token with their tokens taken from a device buffer (as
    the generation loop feeds the sampler's choices back): from the second such step on the
    engine lays nothing out on the host; a kernel moves positions and lengths up by one.  70
    steps cross a page border (and leave a window's pages behind); the logits equal the plain
    implementation's, and a step of another shape in between falls back to the host's layout."""
    import torch
    a, b = _requests(tiny, [90, 80], 51)
    sa, sb = tiny.engine.start_sequences(2)
    out = tiny.step_np([sa, sb], [a[:10], b[:5]], "last")
    got = {0: [out[0:1]], 1: [out[1:2]]}
    src = torch.zeros(2, dtype=torch.int32, device="cuda:0")
    before = tiny.engine.steps_advanced_on_device
    for i in range(70):
        src.copy_(torch.tensor([a[10 + i], b[5 + i]], dtype=torch.int32))
        out = tiny.engine.step([sa, sb], None, "last", from_device=(src, [0, 1])).float().cpu().numpy().copy()
        got[0].append(out[0:1]); got[1].append(out[1:2])
    assert tiny.engine.steps_advanced_on_device - before == 69
    # a step laid out on the host in between, then the device-fed steps again
    out = tiny.step_np([sa, sb], [[a[80]], [b[75]]], "last")
    got[0].append(out[0:1]); got[1].append(out[1:2])
    for i in range(2):
        src.copy_(torch.tensor([a[81 + i], b[76 + i]], dtype=torch.int32))
        out = tiny.engine.step([sa, sb], None, "last", from_device=(src, [0, 1])).float().cpu().numpy().copy()
        got[0].append(out[0:1]); got[1].append(out[1:2])
    assert tiny.engine.steps_advanced_on_device - before == 70
    tiny.engine.cache.check()
    tiny.engine.end_sequences([sa, sb])
    ref_a, ref_b = tiny.reference(a[:83]), tiny.reference(b[:78])
    assert_close(np.concatenate(got[0]), ref_a[9:], tiny.dtype, "first sequence")
    assert_close(np.concatenate(got[1]), ref_b[4:], tiny.dtype, "second sequence")


def test_rows_that_end_are_dropped_on_the_device(tiny):
    """Five sequences decode with their tokens taken from a device buffer.  Two of them end, then the
    rest take their tokens from other places of the buffer, then one more ends and the order of the
    rows is turned round: the engine makes each such step's arrays with a kernel from the step
    before (no layout on the host, nothing copied but page-table rows), and every sequence's logits
    are the plain implementation's."""
    import torch
    lens = [70, 66, 90, 40, 75]
    reqs = _requests(tiny, lens, 61)
    slots = tiny.engine.start_sequences(5)
    pre = [30, 3, 64, 20, 1]
    out = tiny.step_np(slots, [r[:p] for r, p in zip(reqs, pre)], "last")
    got = {i: [out[i:i + 1]] for i in range(5)}
    fed = list(pre)
    src = torch.zeros(8, dtype=torch.int32, device="cuda:0")

    def run(rows, places):
        vals = [0] * 8
        for i, pl in zip(rows, places):
            vals[pl] = reqs[i][fed[i]]
        src.copy_(torch.tensor(vals, dtype=torch.int32))
        o = tiny.engine.step([slots[i] for i in rows], None, "last", from_device=(src, places))
        o = o.float().cpu().numpy().copy()
        for j, i in enumerate(rows):
            got[i].append(o[j:j + 1])
            fed[i] += 1

    eng = tiny.engine
    run([0, 1, 2, 3, 4], [0, 1, 2, 3, 4])            # laid out on the host
    staged, copied, regrouped = eng.stager.staged, eng.stager.bytes_copied, eng.steps_regrouped_on_device
    for _ in range(3):
        run([0, 1, 2, 3, 4], [0, 1, 2, 3, 4])        # advanced
    eng.end_sequences([slots[1], slots[3]])
    run([0, 2, 4], [0, 2, 4])                        # two rows fewer
    run([0, 2, 4], [0, 1, 2])                        # the same rows, other places
    for _ in range(12):
        run([0, 2, 4], [0, 1, 2])                    # advanced (sequence 2 takes a new page on the way)
    eng.end_sequences([slots[0]])
    run([4, 2], [7, 5])                              # one fewer, and the other way round
    for _ in range(5):
        run([4, 2], [7, 5])
    assert eng.steps_regrouped_on_device - regrouped == 3
    assert eng.stager.bytes_copied == copied, "a step was laid out on the host"
    assert eng.stager.staged - staged == 3
    eng.cache.check()
    eng.end_sequences([slots[2], slots[4]])
    for i in range(5):
        assert_close(np.concatenate(got[i]), tiny.reference(reqs[i][:fed[i]])[pre[i] - 1:], tiny.dtype,
                     f"sequence {i}")


def test_one_long_sequence_beside_short_ones(tiny, monkeypatch):
    """Decoding a sequence of 500 tokens together with five of a few tokens, twice: as the engine plans
    it, and with the decode attention told to give a block two pages whatever the sequence (what it
    does by itself where that pays: the long sequence then has four blocks that work, and the short
    ones' surplus blocks write empty partial results).  Every sequence's logits are the plain
    implementation's both times, through the recorded graph too."""
    from torchless_rs_b200.csrc import attention_bf16
    lens = [500, 3, 70, 1, 100, 20]
    reqs = _requests(tiny, [n + 6 for n in lens], 71)
    for forced in (False, True):
        if forced:
            splits_of = attention_bf16.decode_splits
            # (the kernel for head size 32 has no page quantum: it is asked without the lengths)
            monkeypatch.setattr(attention_bf16, "decode_plan",
                                lambda *a: (6, 2) if len(a) > 6 and a[6] is not None else (splits_of(*a[:6]), 0))
            tiny.engine._graphs.clear()
            tiny.engine._seen.clear()
        slots = tiny.engine.start_sequences(len(lens))
        got = [[] for _ in lens]
        tiny.step_np(slots, [r[:n] for r, n in zip(reqs, lens)], "last")
        for step in range(6):
            out = tiny.step_np(slots, [[r[n + step]] for r, n in zip(reqs, lens)], "last")
            for i in range(len(lens)):
                got[i].append(out[i:i + 1])
        tiny.engine.cache.check()
        tiny.engine.end_sequences(slots)
        for i, (r, n) in enumerate(zip(reqs, lens)):
            assert_close(np.concatenate(got[i]), tiny.reference(r)[n:n + 6], tiny.dtype,
                         f"sequence {i} of {n} tokens, {'two pages a block' if forced else 'as planned'}")
    monkeypatch.undo()
    tiny.engine._graphs.clear()
    tiny.engine._seen.clear()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window", [None, 1500])
def test_long_context(dtype, window):
    """A prompt of 2500 tokens in two chunks (2000 + 500: dozens of pages per sequence, the window's
    edge inside the prompt, pages given back between the chunks), a short second sequence beside it,
    then 40 tokens decoded one by one at a context where the keys of a sequence are shared among
    many blocks."""
    from tiny import TINY_D
    cfg = dict(TINY_D, sliding_window=window)
    tm = TinyModel("long", dtype, seed=77, max_tokens=4096, cfg=cfg)
    a, b = _requests(tm, [2540, 75], 61)
    sa, sb = tm.engine.start_sequences(2)
    got_a = [tm.step_np([sa], [a[:2000]], "all")[-50:]]
    out = tm.step_np([sa, sb], [a[2000:2500], b[:35]], "all")
    got_a.append(out[:500]); got_b = [out[500:]]
    for i in range(40):
        out = tm.step_np([sa, sb], [[a[2500 + i]], [b[35 + i]]], "last")
        got_a.append(out[0:1]); got_b.append(out[1:2])
    tm.engine.cache.check()
    if window:
        g = tm.engine.cache.paged[0]
        assert g.first_live[sa] == (2540 - window + 1) // 64     # the pages before the window went back
    tm.engine.end_sequences([sa, sb])
    ref_a, ref_b = tm.reference(a), tm.reference(b)
    assert_close(np.concatenate(got_a), ref_a[1950:], dtype, "long sequence")
    assert_close(np.concatenate(got_b), ref_b, dtype, "short sequence beside it")
