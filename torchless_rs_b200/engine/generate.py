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

from ..sampling.params import SamplingParams, uniform_for

PAGE = 64


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


def generate(engine, select: Callable, prompts: Sequence[Sequence[int]], max_tokens: int,
             params: SamplingParams = SamplingParams(), stop_ids: Sequence[int] = (),
             seed: int = 0, on_token: Optional[Callable[[int, int], None]] = None,
             cache_tokens: Optional[int] = None, max_batch: Optional[int] = None,
             to_host: Callable = lambda t: t.tolist()) -> List[GenerationResult]:
    """Generates up to `max_tokens` tokens for every prompt (lists of token ids).

    A stop token ends its sequence and is not part of the result
    (src/sampler/mod.rs:289-294).  `on_token(request index, token)` is called for
    every emitted token.  The uniform number of a draw depends on (seed, request
    index, number of tokens generated so far), not on how requests were batched."""
    if max_tokens < 0:
        raise ValueError("max_tokens must be >= 0")
    for i, p in enumerate(prompts):
        if len(p) == 0:
            raise ValueError(f"request {i}: the prompt is empty")
    stop = set(int(t) for t in stop_ids)
    results = [GenerationResult(prompt_len=len(p)) for p in prompts]
    if max_tokens == 0 or not prompts:
        return results
    cache_tokens = cache_tokens if cache_tokens is not None else engine.cache.max_tokens
    max_batch = max_batch if max_batch is not None else engine.cache.max_slots
    for batch in plan_batches([len(p) for p in prompts], max_tokens, cache_tokens, max_batch):
        slots = engine.start_sequences(len(batch))
        live = list(zip(batch, slots))          # (request index, slot), in request order
        feed = [list(prompts[i]) for i in batch]
        try:
            while live:
                logits = engine.step([s for _, s in live], feed, want="last")
                uniforms = None
                if not params.is_greedy:
                    uniforms = [uniform_for(seed, i, len(results[i].tokens)) for i, _ in live]
                chosen = to_host(select(logits, params, uniforms))
                nxt_live, feed, ended = [], [], []
                for (i, s), tok in zip(live, chosen):
                    r = results[i]
                    tok = int(tok)
                    if tok in stop:
                        r.stopped_at_eos = True
                        ended.append(s)
                        continue
                    r.tokens.append(tok)
                    if on_token is not None:
                        on_token(i, tok)
                    if len(r.tokens) >= max_tokens:
                        ended.append(s)
                        continue
                    r.steps += 1
                    nxt_live.append((i, s))
                    feed.append([tok])
                if ended:
                    engine.end_sequences(ended)   # ends earlier: its slot is free at once
                live = nxt_live
        except BaseException:
            held = [s for _, s in live]
            if held:
                engine.end_sequences(held)
            raise
    return results
