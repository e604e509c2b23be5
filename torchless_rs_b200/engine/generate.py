"""The generation loop above the step function.

The reference generates for one sequence: forward, sample, stop at an end token
without emitting it, at most `max_tokens` tokens (src/sampler/mod.rs:269-305); its
single-shot command feeds the prompt and then samples from the last prompt token's
logits (src/main.rs:557-598).  Here many requests are served: they are cut into
batches that fit the cache, each batch starts together (prompts of unequal lengths
in one step), a sequence that ends leaves the batch and gives its slot back at once,
and the next batch uses the slots again.

The decisions (how requests are cut into batches, who goes on, who stops) are taken
by plain Python over token ids, so they can be followed without a device: `generate`
only needs an object with `start_sequences`, `end_sequences` and `step`, and a
`select(logits, params, uniforms)` function."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, List, Optional, Sequence

from ..csrc.build import PAGE_TOKENS
from ..sampling.params import SamplingParams, uniform_for

PAGE = PAGE_TOKENS


@dataclass
class GenerationResult:
    """The reference's `GenerationResult {tokens, stopped_at_eos}`
    (src/sampler/mod.rs:257-262) plus the prompt's length and the decode steps run."""
    tokens: List[int] = field(default_factory=list)
    stopped_at_eos: bool = False
    prompt_len: int = 0
    steps: int = 0


def _held(prompt_len: int, max_tokens: int) -> int:
    """Cache tokens a request can come to hold, rounded up to whole pages.  The last
    generated token is never fed back, so it is not held."""
    n = prompt_len + max(max_tokens - 1, 0)
    return (n + PAGE - 1) // PAGE * PAGE


def plan_batches(prompt_lens: Sequence[int], max_tokens: int, cache_tokens: int,
                 max_batch: int) -> List[List[int]]:
    """Cuts requests, in their order, into consecutive batches such that each batch
    has at most `max_batch` sequences and can never hold more than `cache_tokens`
    tokens.  A request that cannot fit alone is an error."""
    batches: List[List[int]] = []
    cur: List[int] = []
    used = 0
    for i, n in enumerate(prompt_lens):
        need = _held(n, max_tokens)
        if need > cache_tokens:
            raise ValueError(
                f"request {i}: a prompt of {n} tokens plus {max_tokens} generated tokens needs "
                f"{need} cache tokens, the cache holds {cache_tokens}")
        if cur and (len(cur) >= max_batch or used + need > cache_tokens):
            batches.append(cur)
            cur, used = [], 0
        cur.append(i)
        used += need
    if cur:
        batches.append(cur)
    return batches


class SyncReader:
    """Brings selected tokens to the host at once (`to_host` turns what `select` returned
    into a list of ints)."""
    overlapped = False

    def __init__(self, to_host: Callable = lambda t: t.tolist()):
        self.to_host = to_host

    def start(self, selected):
        return selected

    def finish(self, handle) -> List[int]:
        return [int(t) for t in self.to_host(handle)]


def generate(engine, select: Callable, prompts: Sequence[Sequence[int]], max_tokens: int,
             params: SamplingParams = SamplingParams(), stop_ids: Sequence[int] = (),
             seed: int = 0, on_token: Optional[Callable[[int, int], None]] = None,
             cache_tokens: Optional[int] = None, max_batch: Optional[int] = None,
             to_host: Callable = lambda t: t.tolist(), reader=None) -> List[GenerationResult]:
    """Generates up to `max_tokens` tokens for every prompt (lists of token ids).

    A stop token ends its sequence and is not part of the result
    (src/sampler/mod.rs:289-294).  `on_token(request index, token)` is called for
    every emitted token.  The uniform number of a draw depends on (seed, request
    index, number of tokens generated so far), not on how requests were batched.

    `reader` brings the selected tokens of a step to the host: `start(selected)` and
    `finish(handle) -> list`.  If it says `overlapped` and the engine's `step` takes
    `from_device`, the next step is launched with the tokens still on the device and the
    host reads them while that step runs; a sequence that turns out to have ended then
    has run one step too many, whose result is dropped."""
    if max_tokens < 0:
        raise ValueError("max_tokens must be >= 0")
    for i, p in enumerate(prompts):
        if len(p) == 0:
            raise ValueError(f"request {i}: the prompt is empty")
    stop = set(int(t) for t in stop_ids)
    results = [GenerationResult(prompt_len=len(p)) for p in prompts]
    if max_tokens == 0 or not prompts:
        return results
    reader = reader if reader is not None else SyncReader(to_host)
    ahead = bool(getattr(reader, "overlapped", False)) and bool(getattr(engine, "takes_device_tokens", False))
    cache_tokens = cache_tokens if cache_tokens is not None else engine.cache.max_tokens
    max_batch = max_batch if max_batch is not None else engine.cache.max_slots

    def uniforms_for(reqs, extra: int):
        if params.is_greedy:
            return None
        return [uniform_for(seed, i, len(results[i].tokens) + extra) for i in reqs]

    def take(i: int, tok: int) -> bool:
        """Books one selected token of request i; True if the sequence goes on."""
        r = results[i]
        if tok in stop:
            r.stopped_at_eos = True
            return False
        r.tokens.append(tok)
        if on_token is not None:
            on_token(i, tok)
        return len(r.tokens) < max_tokens

    for batch in plan_batches([len(p) for p in prompts], max_tokens, cache_tokens, max_batch):
        slots = engine.start_sequences(len(batch))
        held = set(slots)

        def end(ss):
            ss = [s for s in ss if s in held]
            if ss:
                held.difference_update(ss)
                engine.end_sequences(ss)   # ends earlier: its slot is free at once
        try:
            live = list(zip(batch, slots))          # (request index, slot), in request order
            # an engine that offers `prefill` feeds long prompts in several steps (same logits)
            feed = getattr(engine, "prefill", None)
            if feed is not None:
                logits = feed([s for _, s in live], [list(prompts[i]) for i in batch])
            else:
                logits = engine.step([s for _, s in live], [list(prompts[i]) for i in batch], want="last")
            selected = select(logits, params, uniforms_for([i for i, _ in live], 0))
            handle = reader.start(selected)
            where = list(range(len(live)))          # place of each live sequence in `selected`
            while live:
                launched = None
                if ahead:
                    # every sequence that can still go on runs its next step now, fed from the
                    # device; whether its last token was a stop token is learnt below
                    cand = [(w, i, s) for w, (i, s) in zip(where, live)
                            if len(results[i].tokens) + 1 < max_tokens]
                    if cand:
                        logits = engine.step([s for _, _, s in cand], None, want="last",
                                             from_device=(selected, [w for w, _, _ in cand]))
                        nxt = select(logits, params, uniforms_for([i for _, i, _ in cand], 1))
                        launched = (cand, nxt, reader.start(nxt))
                toks = reader.finish(handle)
                going, ended = {}, []
                for w, (i, s) in zip(where, live):
                    if take(i, toks[w]):
                        going[i] = s
                    else:
                        ended.append(s)
                end(ended)
                if ahead:
                    if launched is None:
                        end(list(going.values()))
                        break
                    cand, selected, handle = launched
                    live, where = [], []
                    for place, (_, i, s) in enumerate(cand):
                        if i in going:
                            results[i].steps += 1
                            live.append((i, s))
                            where.append(place)
                else:
                    live = list(going.items())
                    if not live:
                        break
                    for i, _ in live:
                        results[i].steps += 1
                    logits = engine.step([s for _, s in live], [[results[i].tokens[-1]] for i, _ in live],
                                         want="last")
                    selected = select(logits, params, uniforms_for([i for i, _ in live], 0))
                    handle = reader.start(selected)
                    where = list(range(len(live)))
            end(list(held))
        except BaseException:
            if held:
                engine.end_sequences(list(held))
            raise
    return results
