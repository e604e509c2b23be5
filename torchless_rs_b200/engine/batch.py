"""The tokens of one step and where they belong, as the kernels read them."""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence

import numpy as np
import torch


@dataclass
class StepBatch:
    """Packed tokens of all sequences of a step, sequence after sequence.

    Device tensors (int32): `tokens` [T]; `token_seq` [T], the batch row of each
    token; `token_pos` [T], its position in its sequence; `seq_slot` [B], the cache
    slot of each row; `seq_start` [B+1], offsets of the rows in the packed tokens;
    `seq_len` [B], each sequence's length after this step; `want_rows` [R], packed
    indices whose logits are wanted."""
    n_tokens: int
    n_seqs: int
    n_want: int
    is_decode: bool
    max_new: int
    max_len: int
    len_bucket: int       # max_len rounded up to a power of two (at least 256)
    tokens: torch.Tensor
    token_seq: torch.Tensor
    token_pos: torch.Tensor
    seq_slot: torch.Tensor
    seq_start: torch.Tensor
    seq_len: torch.Tensor
    want_rows: torch.Tensor
    token_from: torch.Tensor     # [T] index into `token_src`, or -1 for "use tokens[t]"
    slots: List[int]
    past_lens: List[int]
    new_lens: List[int]
    token_src: Optional[torch.Tensor] = None   # device int32: tokens selected by the previous step
    total_bucket: Optional[int] = None           # the sum of the sequences' lengths after this step, rounded up


def length_bucket(max_len: int) -> int:
    """The longest sequence's length rounded up to a power of two (at least 256)."""
    return max(256, 1 << max(max_len - 1, 0).bit_length())


def total_bucket(lens: Sequence[int]) -> int:
    """The sum of the lengths rounded up to the next of 1, 1.25, 1.5, 1.75 times a power of two (at least
    256): what a recorded decode step may assume about how the keys are spread over the sequences."""
    total = int(sum(lens))
    if total <= 256:
        return 256
    base = 1 << ((total - 1).bit_length() - 1)       # base < total <= 2 base
    for q in (5, 6, 7, 8):
        if total <= base * q // 4:
            return base * q // 4
    return 2 * base


def layout_step(past_lens: Sequence[int], counts: Sequence[int], slots: Sequence[int],
                tokens: Sequence[Sequence[int]], want: Sequence[Sequence[int]]) -> dict:
    """Host arithmetic of a step as numpy arrays (no device needed)."""
    B = len(slots)
    T = int(sum(counts))
    seq_start = np.zeros(B + 1, dtype=np.int32)
    seq_start[1:] = np.cumsum(counts)
    token_seq = np.repeat(np.arange(B, dtype=np.int32), counts)
    token_pos = np.concatenate(
        [np.arange(p, p + c, dtype=np.int32) for p, c in zip(past_lens, counts)]
    ) if T else np.zeros(0, dtype=np.int32)
    toks = np.concatenate([np.asarray(t, dtype=np.int64) for t in tokens]) if T else np.zeros(0, dtype=np.int64)
    want_rows = []
    for b, w in enumerate(want):
        for i in w:
            if not 0 <= i < counts[b]:
                raise ValueError(f"wanted place {i} lies outside the {counts[b]} tokens of entry {b}")
            want_rows.append(int(seq_start[b]) + int(i))
    return dict(
        tokens=toks.astype(np.int32), token_seq=token_seq, token_pos=token_pos,
        seq_slot=np.asarray(slots, dtype=np.int32), seq_start=seq_start,
        seq_len=np.asarray([p + c for p, c in zip(past_lens, counts)], dtype=np.int32),
        want_rows=np.asarray(want_rows, dtype=np.int32),
        token_from=np.full(T, -1, dtype=np.int32))


class BatchStager:
    """Packs a step's arrays into one pinned host buffer and brings them to the
    device with one copy.  The device buffer keeps its address, so views taken for
    the same sizes stay valid from step to step."""

    FIELDS = ("tokens", "token_seq", "token_pos", "seq_slot", "seq_start", "seq_len", "want_rows",
              "token_from")

    RING = 4   # pinned buffers in rotation, so the host can prepare a step while earlier copies run

    def __init__(self, device: torch.device):
        self.device = device
        self.capacity = 0
        self.hosts: List[torch.Tensor] = []
        self.events: List[Optional[torch.cuda.Event]] = []
        self.turn = 0
        self.staged = 0      # steps laid out so far: the device buffer holds the last one's arrays
        self.bytes_copied = 0   # host-to-device bytes of all step layouts so far
        self.dev: Optional[torch.Tensor] = None

    def _ensure(self, n: int) -> None:
        if n <= self.capacity:
            return
        cap = max(4096, 1 << (n - 1).bit_length())
        if self.capacity:
            torch.cuda.synchronize(self.device)
        self.hosts = [torch.empty(cap, dtype=torch.int32, pin_memory=True) for _ in range(self.RING)]
        self.events = [None] * self.RING
        self.dev = torch.empty(cap, dtype=torch.int32, device=self.device)
        self.capacity = cap

    @staticmethod
    def _offsets(sizes):
        """Where each field starts in the buffer: on a 4-element (16-byte) boundary."""
        offs, total = [], 0
        for s in sizes:
            offs.append(total)
            total += (s + 3) // 4 * 4
        return offs, total

    def regroup(self, before: StepBatch, keep, token_from, slots, past_lens, new_lens, ops) -> StepBatch:
        """The decode step of the rows `keep` of the decode step `before`, whose arrays the device buffer
        still holds: a kernel writes the new step's arrays from them (nothing is copied from the host).
        Row j takes its token from place token_from[j] of the sampler's output."""
        n = len(keep)
        sizes = [n, n, n, n, n + 1, n, n, n]
        offs, total = self._offsets(sizes)
        self._ensure(max(total, 1))
        self.staged += 1
        ops.regroup_step(before.token_pos, before.seq_len, before.seq_slot, self.dev, offs, keep, token_from)
        views = {f: self.dev[o:o + s] for f, o, s in zip(self.FIELDS, offs, sizes)}
        max_len = max(new_lens)
        return StepBatch(
            n_tokens=n, n_seqs=n, n_want=n, is_decode=True, max_new=1, max_len=max_len,
            len_bucket=length_bucket(max_len), total_bucket=total_bucket(new_lens),
            slots=list(slots), past_lens=list(past_lens), new_lens=list(new_lens), **views)

    def stage(self, arrays: dict, slots, past_lens, is_decode: bool) -> StepBatch:
        sizes = [int(arrays[f].shape[0]) for f in self.FIELDS]
        offs, total = self._offsets(sizes)
        self._ensure(max(total, 1))
        self.staged += 1
        self.turn = (self.turn + 1) % self.RING
        if self.events[self.turn] is not None:
            self.events[self.turn].synchronize()   # the copy that last used this buffer is done
        host = self.hosts[self.turn]
        hv = host.numpy()
        for f, o, s in zip(self.FIELDS, offs, sizes):
            hv[o:o + s] = arrays[f]
        self.dev[:total].copy_(host[:total], non_blocking=True)
        self.bytes_copied += 4 * total
        ev = self.events[self.turn] or torch.cuda.Event()
        ev.record()
        self.events[self.turn] = ev
        views = {f: self.dev[o:o + s] for f, o, s in zip(self.FIELDS, offs, sizes)}
        counts = np.diff(arrays["seq_start"])
        max_len = int(arrays["seq_len"].max()) if sizes[5] else 0
        return StepBatch(
            n_tokens=sizes[0], n_seqs=sizes[3], n_want=sizes[6], is_decode=is_decode,
            max_new=int(counts.max()) if len(counts) else 0,
            max_len=max_len, len_bucket=length_bucket(max_len),
            total_bucket=total_bucket([int(x) for x in arrays["seq_len"]]),
            slots=list(slots), past_lens=list(past_lens),
            new_lens=[int(x) for x in arrays["seq_len"]], **views)
