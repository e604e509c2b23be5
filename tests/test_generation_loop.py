"""The generation loop's decisions, followed with a scripted engine (no device
needed): batches cut to fit, unequal prompts started together, stop tokens, sequences
that end earlier and give their slot back, slots used again by the next batch."""
import pytest

from torchless_rs_b200.engine.generate import generate, plan_batches
from torchless_rs_b200.sampling.params import SamplingParams, uniform_for


class ScriptedEngine:
    """Stands in for the engine.  The 'logits' of a step are the request-independent
    pairs (slot, position); `select` turns them into tokens with a rule known to the test."""

    def __init__(self, n_slots):
        self.free = list(range(n_slots))
        self.held = set()
        self.length = {}
        self.log = []          # ("start", slots) / ("step", slots, token lists) / ("end", slots)
        self.max_held = 0

    def start_sequences(self, n):
        assert n <= len(self.free), "more sequences started than slots"
        got = [self.free.pop(0) for _ in range(n)]
        self.held.update(got)
        self.max_held = max(self.max_held, len(self.held))
        for s in got:
            self.length[s] = 0
        self.log.append(("start", tuple(got)))
        return got

    def end_sequences(self, slots):
        for s in slots:
            assert s in self.held, "slot given back twice"
            self.held.remove(s)
        self.free = sorted(self.free + list(slots))
        self.log.append(("end", tuple(slots)))

    def step(self, slots, tokens, want="last", from_device=None):
        if from_device is not None:
            src, idx = from_device
            tokens = [[src[j]] for j in idx]
        assert want == "last" and len(slots) == len(tokens)
        for s, t in zip(slots, tokens):
            assert s in self.held
            self.length[s] += len(t)
        self.log.append(("step", tuple(slots), tuple(len(t) for t in tokens)))
        return [(s, self.length[s], t[-1]) for s, t in zip(slots, tokens)]


def next_token(last_token, length):
    return (last_token * 7 + length) % 50


def select(logits, params, uniforms):
    return [next_token(last, length) for _, length, last in logits]


def expected(prompt, max_tokens, stop):
    seq, out = list(prompt), []
    for _ in range(max_tokens):
        t = next_token(seq[-1], len(seq))
        if t in stop:
            return out, True
        out.append(t)
        seq.append(t)
    return out, False


def test_plan_batches_fits_the_cache():
    assert plan_batches([5, 11, 23], 8, 64 * 3, 8) == [[0, 1, 2]]
    assert plan_batches([5, 11, 23], 8, 64 * 2, 8) == [[0, 1], [2]]
    assert plan_batches([5, 11, 23, 7, 9], 8, 10 ** 6, 2) == [[0, 1], [2, 3], [4]]
    assert plan_batches([60, 60], 6, 128, 8) == [[0], [1]]    # 60 + 5 held tokens need two pages each
    assert plan_batches([60, 60], 5, 128, 8) == [[0, 1]]      # the last token is never fed back
    with pytest.raises(ValueError, match="request 1"):
        plan_batches([5, 500], 8, 256, 8)


def test_unequal_prompts_stop_tokens_and_early_enders():
    prompts = [[1, 2, 3, 4, 5], [9], [7, 7, 7], [4, 4], [30, 2, 2, 2, 2, 2, 2]]
    stop = {13, 21}
    eng = ScriptedEngine(n_slots=2)
    seen = []
    res = generate(eng, select, prompts, 12, SamplingParams.greedy(), stop, on_token=lambda i, t: seen.append((i, t)),
                   cache_tokens=10 ** 6, max_batch=2, to_host=list)
    for i, p in enumerate(prompts):
        toks, stopped = expected(p, 12, stop)
        assert res[i].tokens == toks and res[i].stopped_at_eos == stopped, i
        assert res[i].prompt_len == len(p)
        assert [t for j, t in seen if j == i] == toks
    assert any(r.stopped_at_eos for r in res) and any(not r.stopped_at_eos for r in res)
    assert eng.max_held <= 2 and not eng.held            # nothing leaks
    starts = [e for e in eng.log if e[0] == "start"]
    assert [len(e[1]) for e in starts] == [2, 2, 1]       # three batches, one after another
    assert starts[0][1] == starts[1][1]                   # the same slots again
    # the first step of a batch carries whole prompts of unequal length, later steps one token each
    first = eng.log[1]
    assert first[0] == "step" and first[2] == (5, 1)
    later = [e for e in eng.log if e[0] == "step" and e is not first and e[1] == first[1]]
    assert all(set(e[2]) == {1} for e in later[:1])


def test_a_sequence_that_ends_leaves_the_batch_at_once():
    prompts = [[1], [2]]
    eng = ScriptedEngine(2)
    res = generate(eng, select, prompts, 30, SamplingParams.greedy(), {13, 21, 40}, cache_tokens=10 ** 6,
                   max_batch=2, to_host=list)
    n0, n1 = len(res[0].tokens), len(res[1].tokens)
    assert n0 != n1
    steps = [e for e in eng.log if e[0] == "step"]
    assert len(steps[0][1]) == 2 and len(steps[-1][1]) == 1     # the batch shrinks
    ends = [e for e in eng.log if e[0] == "end"]
    assert len(ends) == 2 and eng.log.index(ends[0]) < len(eng.log) - 1


def test_max_tokens_and_empty_cases():
    eng = ScriptedEngine(4)
    res = generate(eng, select, [[3, 3]], 0, cache_tokens=1024, max_batch=4, to_host=list)
    assert res[0].tokens == [] and eng.log == []
    res = generate(eng, select, [[3, 3]], 1, stop_ids=(), cache_tokens=1024, max_batch=4, to_host=list)
    assert len(res[0].tokens) == 1 and res[0].steps == 0
    assert [e[0] for e in eng.log] == ["start", "step", "end"]   # the last token is never fed back
    with pytest.raises(ValueError, match="empty"):
        generate(eng, select, [[]], 3, cache_tokens=1024, max_batch=4, to_host=list)


def test_slots_come_back_when_a_step_fails():
    class Failing(ScriptedEngine):
        def step(self, slots, tokens, want="last"):
            if len(self.log) > 3:
                raise RuntimeError("boom")
            return super().step(slots, tokens, want)
    eng = Failing(2)
    with pytest.raises(RuntimeError, match="boom"):
        generate(eng, select, [[1], [2]], 20, stop_ids=(), cache_tokens=10 ** 6, max_batch=2, to_host=list)
    assert not eng.held


def test_uniform_numbers_do_not_depend_on_batching():
    got = []

    def sel(logits, params, uniforms):
        got.append(tuple(uniforms))
        return select(logits, params, uniforms)
    prompts = [[1], [2], [3]]
    for mb in (1, 3):
        got.clear()
        generate(ScriptedEngine(3), sel, prompts, 3, SamplingParams(temperature=0.8), (), seed=5,
                 cache_tokens=10 ** 6, max_batch=mb, to_host=list)
        flat = sorted(u for row in got for u in row)
        want = sorted(uniform_for(5, i, k) for i in range(3) for k in range(3))
        assert flat == want
    assert 0.0 <= uniform_for(1, 2, 3) < 1.0 and uniform_for(1, 2, 3) != uniform_for(1, 2, 4)


class AheadReader:
    """Says that reading may overlap the next step; here both ends are immediate."""
    overlapped = True

    def start(self, selected):
        return list(selected)

    def finish(self, handle):
        return handle


def test_one_step_ahead_gives_the_same_tokens_and_at_most_one_extra_step():
    prompts = [[1, 2, 3, 4, 5], [9], [7, 7, 7], [4, 4], [30, 2, 2, 2, 2, 2, 2]]
    stop = {13, 21}
    for mb in (2, 5):
        eng = ScriptedEngine(n_slots=mb)
        eng.takes_device_tokens = True
        res = generate(eng, select, prompts, 12, SamplingParams.greedy(), stop, cache_tokens=10 ** 6,
                       max_batch=mb, reader=AheadReader())
        for i, p in enumerate(prompts):
            toks, stopped = expected(p, 12, stop)
            assert res[i].tokens == toks and res[i].stopped_at_eos == stopped, (mb, i)
        assert not eng.held
        # a sequence runs one step per token it feeds back; one more only if a stop token
        # ended it (learnt one step late); never beyond max_tokens
        fed = {}
        slot_req = {}
        for e in eng.log:
            if e[0] == "start":
                starts = e[1]
            if e[0] == "step":
                for s_ in e[1]:
                    fed[s_] = fed.get(s_, 0) + 1
        total_steps = sum(len(e[1]) for e in eng.log if e[0] == "step")
        needed = sum(1 + max(len(r.tokens) - (0 if r.stopped_at_eos else 1), 0) for r in res)
        extra = total_steps - needed
        assert 0 <= extra <= sum(1 for r in res if r.stopped_at_eos), (mb, extra)


def test_ahead_with_sampling_uses_the_same_uniform_numbers():
    got = {}

    def sel(logits, params, uniforms):
        for (slot, length, last), u in zip(logits, uniforms):
            got.setdefault((slot, length), u)
        return select(logits, params, uniforms)
    prompts = [[1], [2, 5], [3]]
    runs = []
    for reader in (None, AheadReader()):
        got.clear()
        eng = ScriptedEngine(3)
        eng.takes_device_tokens = True
        generate(eng, sel, prompts, 4, SamplingParams(temperature=0.8), (), seed=5, cache_tokens=10 ** 6,
                 max_batch=3, reader=reader, to_host=list)
        runs.append(dict(got))
    assert runs[0] == runs[1]


def test_a_set_error_word_is_raised_and_cleared():
    """A kernel library that gave up on a bounded wait leaves a nonzero error word; the check
    that generation and replay make where they wait for results anyway raises it, once."""
    from torchless_rs_b200.csrc import ops

    word = {"v": 0}

    def take():
        v, word["v"] = word["v"], 0
        return v

    ops.register_error_word("toy_library", take)
    try:
        ops.check_kernel_errors()
        word["v"] = 3
        with pytest.raises(ops.KernelError, match="toy_library: code 3"):
            ops.check_kernel_errors()
        ops.check_kernel_errors()
    finally:
        ops._error_words.pop("toy_library")


def test_an_engine_that_offers_prefill_gets_the_prompts_through_it():
    """The loop hands a batch's prompts to `prefill` where the engine has one (it may cut them into
    several steps) and decodes with `step` afterwards; the tokens are the same."""
    class WithPrefill(ScriptedEngine):
        def prefill(self, slots, prompts):
            for a in range(0, max(len(p) for p in prompts), 2):       # two tokens of each prompt a step
                rows = [(s, p[a:a + 2]) for s, p in zip(slots, prompts) if p[a:a + 2]]
                self.step([s for s, _ in rows], [t for _, t in rows])
            return [(s, self.length[s], p[-1]) for s, p in zip(slots, prompts)]

    prompts = [[1, 2, 3, 4, 5], [9], [7, 7, 7]]
    eng = WithPrefill(n_slots=3)
    res = generate(eng, select, prompts, 6, SamplingParams.greedy(), set(), cache_tokens=10 ** 6, max_batch=3,
                   to_host=list)
    for i, p in enumerate(prompts):
        assert res[i].tokens == expected(p, 6, set())[0], i
    steps = [e for e in eng.log if e[0] == "step"]
    assert [e[2] for e in steps[:3]] == [(2, 1, 2), (2, 1), (1,)]      # the prompts, cut
    assert all(set(e[2]) == {1} for e in steps[3:])                    # then one token each
    assert not eng.held
