"""The step function: one batch of sequences, the tokens it is given, from the cache.

The reference's forward takes one token of one sequence and the caller advances
the position (src/model/mod.rs:430-468, src/main.rs:557-563).  Here a step takes a
batch whose sequences either all start (prompts of unequal lengths, run together
as one packed batch) or all go on by one token; positions come from the cache's
record of each sequence and advance inside the step."""
from __future__ import annotations

from typing import List, Optional, Sequence, Union

import numpy as np
import torch

from ..cache import Cache
from ..config.spec import ModelSpec
from ..csrc import ops
from ..parts.runtime import Runtime
from .batch import BatchStager, StepBatch, layout_step, length_bucket, total_bucket
from .model import DecoderModel


class Engine:
    """Owns the model, its cache and the staging of steps.

    `max_tokens`: the most tokens that live sequences hold at any time, each
    sequence's count rounded up to a multiple of 64; it sizes the cache."""

    def __init__(self, spec: ModelSpec, weights, rt: Runtime, max_tokens: int,
                 max_batch: Optional[int] = None, max_seq_len: Optional[int] = None,
                 use_graphs: bool = True):
        self.spec = spec
        self.rt = rt
        self.model = DecoderModel(spec, rt)
        self.model.load(weights)
        if spec.position_table_name is not None:
            # a learned position table has a last row: no sequence may grow past it
            max_seq_len = min(max_seq_len or spec.max_positions, spec.max_positions)
        self.cache = Cache(self.model.cache_requests(), max_tokens, max_batch, max_seq_len,
                           dtype=rt.act_dtype, device=rt.device)
        self.model.bind_cache(self.cache)
        self.stager = BatchStager(rt.device)
        self.vocab_size = spec.vocab_size
        self.takes_device_tokens = True   # step(..., from_device=...) is supported
        self.use_graphs = use_graphs
        self._graphs = {}      # key -> (CUDA graph, logits view)
        self._seen = set()     # keys that have run once without a graph
        self._steady = None    # (key, staged count, batch) of the last decode step fed from the device
        self.steps_advanced_on_device = 0
        self.steps_regrouped_on_device = 0   # decode steps whose rows a kernel chose from the step before

    # ---- sequences -------------------------------------------------------------------
    def start_sequences(self, count: int) -> List[int]:
        """Takes `count` free slots; each stands for a new, empty sequence."""
        return self.cache.acquire(count)

    def end_sequences(self, slots: Sequence[int]) -> None:
        """Gives the slots and everything they hold back."""
        self.cache.release(slots)

    def length(self, slot: int) -> int:
        return self.cache.length(slot)

    def truncate(self, slot: int, length: int) -> None:
        """Shortens a sequence to its first `length` tokens; its next step goes on from there
        (the reference's /retry lowers its position counter the same way, src/main.rs:1722-1726).
        Raises `CacheRollbackError` where that is not possible (see `Cache.truncate`)."""
        self.cache.truncate(slot, length)

    def reset(self, slot: int) -> None:
        """The sequence starts again at its first token (src/model/mod.rs:234-237); the slot
        stays held."""
        self.cache.reset(slot)

    def h2d_bytes(self) -> int:
        """Host-to-device bytes that steps have copied so far: step layouts and page-table rows."""
        return self.stager.bytes_copied + sum(g.bytes_copied for g in self.cache.paged)

    def check_kernels(self) -> None:
        """Raises if a kernel gave up on one of its bounded waits since the last check (its
        results are then wrong).  Synchronises the device."""
        ops.check_kernel_errors()

    # ---- the step ----------------------------------------------------------------------
    def step(self, slots: Sequence[int], tokens: Optional[Sequence[Sequence[int]]] = None,
             want: Union[str, Sequence[Sequence[int]]] = "last",
             from_device=None) -> Optional[torch.Tensor]:
        """Runs `tokens[b]` as the next tokens of the sequence in `slots[b]` and
        returns the 32-bit logits [wanted, vocab] on the device, in the order of the
        sequences and of their wanted places (`want[b]`: indices into `tokens[b]`;
        "last": the last token of each; "all"; "none").  The returned tensor is a
        view of a buffer that the next step overwrites.

        `from_device` = (source, indices) instead of `tokens`: every sequence goes on by the
        one token source[indices[b]], where `source` is an int32 tensor on the device (the
        tokens a sampler selected).  The host then need not know the tokens to launch the step."""
        B = len(slots)
        if B == 0:
            return None
        token_src = None
        if from_device is not None:
            token_src, src_index = from_device
            if len(src_index) != B:
                raise ValueError("one source index per slot is needed")
            tokens = [[0]] * B
        if len(tokens) != B:
            raise ValueError("one token list per slot is needed")
        counts = [len(t) for t in tokens]
        if min(counts) < 1:
            raise ValueError("every sequence of a step brings at least one token")
        if want == "last":
            want = [[c - 1] for c in counts]
        elif want == "all":
            want = [list(range(c)) for c in counts]
        elif want == "none" or want is None:
            want = [[] for _ in counts]
        past = [self.cache.length(s) for s in slots]
        new_lens = [p + c for p, c in zip(past, counts)]
        # The same sequences in the same rows as the decode step before, fed from the device again:
        # only positions and lengths differ, by one, and a kernel advances them on the device; the
        # host lays nothing out and copies nothing but page-table rows that gained a page.
        steady_key = None
        if token_src is not None and all(c == 1 for c in counts) and all(w == [0] for w in want):
            steady_key = (tuple(slots), tuple(int(i) for i in src_index), token_src.data_ptr())
            st = self._steady
            if st is not None and st[0] == steady_key and st[1] == self.stager.staged and \
                    st[2].new_lens == past:
                batch = st[2]
                self.cache.prepare(slots, new_lens)
                self.rt.ops.advance_step(batch.token_pos, batch.seq_len)
                batch.past_lens, batch.new_lens = list(past), list(new_lens)
                batch.max_len = max(new_lens)
                batch.len_bucket = length_bucket(batch.max_len)
                batch.total_bucket = total_bucket(new_lens)
                batch.token_src = token_src
                self.steps_advanced_on_device += 1
                logits = self._forward(batch)
                self.cache.commit(slots, new_lens)
                return logits
            # Some of that step's sequences (others have ended), or the same ones taking their tokens
            # from other places: a kernel makes the new step's arrays from the old ones.
            if st is not None and st[1] == self.stager.staged and B <= self.rt.ops.REGROUP_MAX_ROWS:
                row_of = {s: r for r, s in enumerate(st[2].slots)}
                keep = [row_of.get(s, -1) for s in slots]
                if min(keep) >= 0 and max(keep) < 65536 and len(set(slots)) == B and \
                        all(st[2].new_lens[r] == p for r, p in zip(keep, past)) and \
                        all(0 <= int(i) < 65536 for i in src_index):
                    self.cache.prepare(slots, new_lens)
                    batch = self.stager.regroup(st[2], keep, [int(i) for i in src_index], slots, past,
                                                new_lens, self.rt.ops)
                    batch.token_src = token_src
                    self._steady = (steady_key, self.stager.staged, batch)
                    self.steps_regrouped_on_device += 1
                    logits = self._forward(batch)
                    self.cache.commit(slots, new_lens)
                    return logits
        arrays = layout_step(past, counts, slots, tokens, want)
        if token_src is not None:
            arrays["token_from"] = np.asarray(src_index, dtype=np.int32)
        toks = arrays["tokens"]
        if toks.size and (toks.min() < 0 or toks.max() >= self.vocab_size):
            raise ValueError(f"token ids must lie in [0, {self.vocab_size})")
        self.cache.prepare(slots, new_lens)
        batch = self.stager.stage(arrays, slots, past, is_decode=all(c == 1 for c in counts))
        batch.token_src = token_src
        self._steady = (steady_key, self.stager.staged, batch) if steady_key is not None else None
        logits = self._forward(batch)
        self.cache.commit(slots, new_lens)
        return logits

    # Tokens per step beyond which a batch of prompts is fed in several steps: a bound on the workspace (a
    # step of 65,536 tokens at the layer sizes of Mistral NeMo 12B holds some 6 GB of activations), not a
    # gain in time.  Measured on 8 layers in bfloat16 since the many-token products walk their tiles in
    # groups of weight strips: 8 prompts of 8192 tokens at the NeMo sizes 274 to 277 ms in one step, 274 ms in
    # steps of 16,384 tokens, 277 at 8192, 284 at 4096; 16 prompts of 128 to 4096 tokens at the sizes of Mistral
    # Small 22B 202 to 208 / 201 to 210 / 209 to 216 / 218 ms; one prompt of 16,384 tokens at the 7B sizes 52 /
    # 51 / 56 / 60 ms.  (Before that change one step of 65,536 tokens took 337 ms and steps of 4096 tokens 286:
    # the large step's products read their activations again for every strip of weights.)
    PREFILL_TOKENS_PER_STEP = 65536

    def prefill(self, slots: Sequence[int], prompts: Sequence[Sequence[int]],
                tokens_per_step: Optional[int] = None) -> torch.Tensor:
        """Feeds the prompts of sequences that start together and returns the 32-bit logits
        [sequences, vocab] at each prompt's last token (a buffer of its own, valid until the next
        call).  Prompts whose tokens together exceed `tokens_per_step` are fed in several steps, every
        sequence that still has tokens going on by the same number of them (a multiple of the page
        size, at least 128; a prompt's end up to a quarter more); the result does not depend on the
        cut beyond rounding."""
        B = len(slots)
        if len(prompts) != B:
            raise ValueError("one prompt per slot is needed")
        if any(len(p) == 0 for p in prompts):
            raise ValueError("every sequence of a step brings at least one token")
        budget = tokens_per_step or self.PREFILL_TOKENS_PER_STEP
        total = sum(len(p) for p in prompts)
        if total <= budget:
            return self.step(slots, [list(p) for p in prompts], "last")
        out = self.rt.workspace.get("prefill_logits", (B, self.vocab_size), torch.float32)
        fed = [0] * B
        while True:
            rows = [b for b in range(B) if fed[b] < len(prompts[b])]
            if not rows:
                return out
            # the sequences that still have tokens share the step: when the short prompts have run
            # out, the long ones go on in larger pieces
            chunk = max(128, budget // len(rows) // 64 * 64)
            # a prompt's last tokens do not get a step of their own: up to a quarter more goes now
            toks = [list(prompts[b][fed[b]:fed[b] + (chunk if len(prompts[b]) - fed[b] > chunk + chunk // 4
                                                       else len(prompts[b]))]) for b in rows]
            ends = [fed[b] + len(t) >= len(prompts[b]) for b, t in zip(rows, toks)]
            logits = self.step([slots[b] for b in rows], toks, [[len(t) - 1] if e else [] for t, e in zip(toks, ends)])
            k = 0
            for b, t, e in zip(rows, toks, ends):
                fed[b] += len(t)
                if e:
                    out[b].copy_(logits[k])
                    k += 1

    def _forward(self, batch: StepBatch) -> Optional[torch.Tensor]:
        """Decode steps of one shape launch the same kernels with the same arguments
        (token ids, positions and page tables are read from device memory), so the
        second step of a shape is recorded as a CUDA graph and later ones replay it."""
        if not (self.use_graphs and batch.is_decode and self.model.graph_safe):
            return self.model.forward(batch)
        key = (batch.n_seqs, batch.n_want, batch.len_bucket, batch.total_bucket, self.rt.workspace.generation,
               batch.tokens.data_ptr(), batch.token_src.data_ptr() if batch.token_src is not None else 0)
        hit = self._graphs.get(key)
        if hit is not None:
            hit[0].replay()
            ops.add_launches(hit[3])
            return hit[1]
        if key not in self._seen:
            self._seen.add(key)
            return self.model.forward(batch)
        if len(self._graphs) > 64:
            self._graphs.clear()
        graph = torch.cuda.CUDAGraph()
        torch.cuda.synchronize()
        before = ops.launch_counts()
        with torch.cuda.graph(graph):
            logits = self.model.forward(batch)
        recorded = ops.counts_since(before)   # recording launches nothing; replay runs them all
        ops.add_launches(recorded, -1)
        if self.rt.workspace.generation != key[4]:   # a buffer moved while recording
            return self.model.forward(batch)
        self._graphs[key] = (graph, logits, batch, recorded)
        graph.replay()
        ops.add_launches(recorded)
        return logits
