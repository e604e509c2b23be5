"""The cache of a model: a slot per live sequence, paged keys and values per layer,
and per-sequence state of fixed size.

The reference keeps one tensor [layers, kv_heads, max_seq_len, head_dim] for one
sequence (src/model/kv_cache.rs:23-53) and a position counter that the caller
advances (src/model/mod.rs:93).  Here many sequences live at once:

* a *slot* stands for one sequence; it records the sequence's length and is given
  back when the sequence ends, then used again;
* layers whose mixers ask for the same thing form a *group* with storage of its own.
  A paged group holds keys and values in pages of `PAGE` positions,
  [layers, 2, pages, kv_heads, PAGE * head_dim] (keys as [PAGE, head_dim], values
  transposed as [head_dim, PAGE]), and a table from (slot, position //
  PAGE) to a page.  A group with a window gives pages back as soon as every position
  in them has left the window of the sequence's next position;
* a state group holds [layers, slots, *shape], zeroed when a slot is taken.

All decisions are taken on the host; the device only sees the page tables.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Union

import numpy as np
import torch

from ..csrc.build import PAGE_TOKENS
from .pages import CacheCapacityError, CacheRollbackError, CacheStateError, FreeList
from .requests import PagedKVRequest, StateRequest

PAGE = PAGE_TOKENS   # tokens per cache page: the number the kernels were compiled with


def pages_for(n_tokens: int) -> int:
    return (n_tokens + PAGE - 1) // PAGE


@dataclass
class PagedView:
    """What an attention mixer gets for its layer."""
    k_pages: torch.Tensor       # [pages, kv_heads, PAGE, head_dim]
    v_pages: torch.Tensor       # [pages, kv_heads, head_dim, PAGE]: values lie transposed
    page_table: torch.Tensor    # [slots, pages per sequence] int32, on the device
    window: Optional[int]
    group: "PagedGroup"


class PagedGroup:
    def __init__(self, request: PagedKVRequest, layers: Sequence[int], n_pages: int,
                 max_slots: int, table_width: int, dtype: torch.dtype, device: torch.device):
        self.request = request
        self.layers = list(layers)
        self.n_pages = n_pages
        self.pool = FreeList(n_pages, "cache page")
        self.storage = torch.zeros(
            (len(self.layers), 2, n_pages, request.num_kv_heads, PAGE * request.head_dim),
            dtype=dtype, device=device)
        self.table_host = np.full((max_slots, table_width), -1, dtype=np.int32)
        self.table_dev = torch.full((max_slots, table_width), -1, dtype=torch.int32, device=device)
        self.first_live = [0] * max_slots   # first table column that still holds a page
        self.n_cols = [0] * max_slots       # table columns filled so far
        self._dirty: set = set()
        self.bytes_copied = 0   # host-to-device bytes of page-table rows so far
        # rows on their way to the device are snapshots in pinned memory (several in rotation):
        # the host may change the table again before an earlier copy has run
        self._staging = None
        self._staging_events = []
        self._turn = 0

    def pages_needed(self, slot: int, new_len: int) -> int:
        return max(0, pages_for(new_len) - self.n_cols[slot])

    def grow(self, slot: int, new_len: int) -> None:
        need = self.pages_needed(slot, new_len)
        if need == 0:
            return
        if pages_for(new_len) > self.table_host.shape[1]:
            raise CacheCapacityError(
                f"a sequence of {new_len} tokens is longer than the cache was sized for "
                f"({self.table_host.shape[1] * PAGE})")
        got = self.pool.take(need)
        c = self.n_cols[slot]
        self.table_host[slot, c:c + need] = got
        self.n_cols[slot] = c + need
        self._dirty.add(slot)

    def trim(self, slot: int, next_pos: int) -> None:
        """Gives back the pages that no position >= next_pos can see any more."""
        w = self.request.window
        if not w:
            return
        first_needed_key = max(0, next_pos - w + 1)
        keep_from = min(first_needed_key // PAGE, self.n_cols[slot])
        f = self.first_live[slot]
        if keep_from > f:
            self.pool.give_back(int(p) for p in self.table_host[slot, f:keep_from])
            self.table_host[slot, f:keep_from] = -1
            self.first_live[slot] = keep_from
            self._dirty.add(slot)

    def can_truncate(self, slot: int, new_len: int) -> bool:
        """Whether the keys that position `new_len` will see are still held."""
        w = self.request.window
        if not w or new_len == 0:
            return True
        return max(0, new_len - w + 1) // PAGE >= self.first_live[slot]

    def truncate(self, slot: int, new_len: int) -> None:
        """Gives back the whole pages beyond `new_len` positions.  What lies beyond `new_len`
        in the last kept page stays there; no kernel reads past a sequence's length, and the
        next tokens overwrite it."""
        keep = pages_for(new_len)
        f, c = self.first_live[slot], self.n_cols[slot]
        if keep >= c:
            return
        lo = max(keep, f)
        if c > lo:
            self.pool.give_back(int(p) for p in self.table_host[slot, lo:c])
        self.table_host[slot, keep:c] = -1
        self.n_cols[slot] = keep
        self.first_live[slot] = min(f, keep)
        self._dirty.add(slot)

    def release(self, slot: int) -> None:
        f, c = self.first_live[slot], self.n_cols[slot]
        if c > f:
            self.pool.give_back(int(p) for p in self.table_host[slot, f:c])
        self.table_host[slot, :c] = -1
        self.first_live[slot] = 0
        self.n_cols[slot] = 0
        self._dirty.add(slot)

    def upload(self) -> None:
        if not self._dirty:
            return
        rows = sorted(self._dirty)
        self._dirty.clear()
        if not self.table_dev.is_cuda:
            idx = torch.as_tensor(rows, dtype=torch.long)
            self.table_dev.index_copy_(0, idx, torch.from_numpy(self.table_host[rows]))
            return
        chunk = 32   # rows per snapshot buffer
        if self._staging is None:
            self._staging = torch.empty((4, chunk, self.table_host.shape[1]), dtype=torch.int32,
                                        pin_memory=True)
            self._staging_events = [None] * 4
        for c0 in range(0, len(rows), chunk):
            self._turn = (self._turn + 1) % 4
            if self._staging_events[self._turn] is not None:
                self._staging_events[self._turn].synchronize()
            stage = self._staging[self._turn]
            stage_np = stage.numpy()
            for j, r in enumerate(rows[c0:c0 + chunk]):
                stage_np[j] = self.table_host[r]
                self.table_dev[r].copy_(stage[j], non_blocking=True)
                self.bytes_copied += 4 * self.table_host.shape[1]
            ev = self._staging_events[self._turn] or torch.cuda.Event()
            ev.record()
            self._staging_events[self._turn] = ev

    def view(self, layer: int) -> PagedView:
        i = self.layers.index(layer)
        r = self.request
        k = self.storage[i, 0].view(self.n_pages, r.num_kv_heads, PAGE, r.head_dim)
        v = self.storage[i, 1].view(self.n_pages, r.num_kv_heads, r.head_dim, PAGE)
        return PagedView(k, v, self.table_dev, r.window, self)


class StateGroup:
    def __init__(self, request: StateRequest, layers: Sequence[int], max_slots: int,
                 device: torch.device):
        self.request = request
        self.layers = list(layers)
        self.storage = torch.zeros((len(self.layers), max_slots, *request.shape),
                                   dtype=request.dtype, device=device)

    def reset(self, slot: int) -> None:
        self.storage[:, slot].zero_()

    def view(self, layer: int) -> torch.Tensor:
        """[slots, *shape] of one layer."""
        return self.storage[self.layers.index(layer)]


class Cache:
    """`requests[k]` is what the mixer of the k-th entry of the layer order asks for
    (None: nothing, or it reads another entry's cache); "layer" below means such an entry.  `max_tokens` is the most tokens that live sequences hold
    at any time, each sequence's count rounded up to a multiple of PAGE."""

    def __init__(self, requests: Sequence[Union[PagedKVRequest, StateRequest, None]],
                 max_tokens: int, max_slots: Optional[int] = None,
                 max_seq_len: Optional[int] = None, dtype: torch.dtype = torch.bfloat16,
                 device: Union[str, torch.device] = "cuda"):
        self.device = torch.device(device)
        self.dtype = dtype
        n_pages = max(1, pages_for(max_tokens))
        self.max_tokens = n_pages * PAGE
        self.max_slots = max_slots if max_slots else min(n_pages, 256)
        self.max_seq_len = min(max_seq_len, self.max_tokens) if max_seq_len else self.max_tokens
        table_width = pages_for(self.max_seq_len)
        self.slots = FreeList(self.max_slots, "sequence slot")
        self.lengths = [0] * self.max_slots
        self.paged: List[PagedGroup] = []
        self.states: List[StateGroup] = []
        self._of_layer: Dict[int, Union[PagedGroup, StateGroup]] = {}
        by_request: Dict[object, List[int]] = {}
        for layer, req in enumerate(requests):
            if req is not None:
                by_request.setdefault(req, []).append(layer)
        for req, layers in by_request.items():
            if isinstance(req, PagedKVRequest):
                g = PagedGroup(req, layers, n_pages, self.max_slots, table_width, dtype, self.device)
                self.paged.append(g)
            elif isinstance(req, StateRequest):
                g = StateGroup(req, layers, self.max_slots, self.device)
                self.states.append(g)
            else:
                raise TypeError(f"unknown cache request {req!r}")
            for layer in layers:
                self._of_layer[layer] = g

    # ---- slots -----------------------------------------------------------------
    def acquire(self, count: int = 1) -> List[int]:
        got = self.slots.take(count)
        for s in got:
            self.lengths[s] = 0
            for g in self.states:
                g.reset(s)
        return got

    def release(self, slots) -> None:
        slots = list(slots)
        for s in slots:
            if not self.slots.is_held(s):
                raise CacheStateError(f"sequence slot {s} is released but is not held")
        for s in slots:
            for g in self.paged:
                g.release(s)
            self.lengths[s] = 0
        self.slots.give_back(slots)

    def length(self, slot: int) -> int:
        return self.lengths[slot]

    def truncate(self, slot: int, length: int) -> None:
        """Shortens the sequence of `slot` to its first `length` tokens, so that its next step
        goes on from there.  The reference rolls its one sequence back by lowering the position
        counter (src/main.rs:1722-1726, the chat's /retry; src/model/mod.rs:234-237 for the
        return to zero); here whole pages beyond `length` also go back to the pool.

        Raises `CacheRollbackError`, and changes nothing, if a window has already given back
        keys that position `length` would see, or if `length` > 0 and a mixer keeps state of
        fixed size.  `length` = 0 is always possible: pages are given back and state is zeroed."""
        if not self.slots.is_held(slot):
            raise CacheStateError(f"sequence slot {slot} is shortened but is not held")
        cur = self.lengths[slot]
        if not 0 <= length <= cur:
            raise ValueError(f"a sequence of {cur} tokens cannot be shortened to {length}")
        if length == cur:
            return
        if length > 0:
            if self.states:
                raise CacheRollbackError(
                    "a mixer of this model keeps per-sequence state of fixed size, which cannot be "
                    "rolled back; only reset (length 0) is possible")
            for g in self.paged:
                if not g.can_truncate(slot, length):
                    w = g.request.window
                    raise CacheRollbackError(
                        f"slot {slot} cannot be shortened from {cur} to {length} tokens: position "
                        f"{length} sees keys from {max(0, length - w + 1)} on, but the window of {w} "
                        f"has already given back everything before {g.first_live[slot] * PAGE}")
        for g in self.paged:
            g.truncate(slot, length)
            g.upload()
        if length == 0:
            for g in self.states:
                g.reset(slot)
        self.lengths[slot] = length

    def reset(self, slot: int) -> None:
        """The sequence of `slot` starts again at its first token; the slot stays held."""
        self.truncate(slot, 0)

    # ---- one step ----------------------------------------------------------------
    def prepare(self, slots: Sequence[int], new_lens: Sequence[int]) -> None:
        """Makes room for each sequence to reach its new length and brings the
        device's page tables up to date.  Nothing changes if there is no room."""
        for s in slots:
            if not self.slots.is_held(s):
                raise CacheStateError(f"sequence slot {s} is used but is not held")
        if len(set(slots)) != len(slots):
            raise CacheStateError("a sequence slot appears twice in one step")
        for s, n in zip(slots, new_lens):
            if n > self.max_seq_len:
                raise CacheCapacityError(
                    f"a sequence of {n} tokens is longer than the cache was sized for "
                    f"({self.max_seq_len})")
        for g in self.paged:
            need = sum(g.pages_needed(s, n) for s, n in zip(slots, new_lens))
            if need > g.pool.free_count:
                raise CacheCapacityError(
                    f"the cache is full: this step needs {need} more pages of {PAGE} tokens, "
                    f"{g.pool.free_count} of {g.n_pages} are free")
        for g in self.paged:
            for s, n in zip(slots, new_lens):
                g.grow(s, n)
            g.upload()

    def commit(self, slots: Sequence[int], new_lens: Sequence[int]) -> None:
        """Records the new lengths after a step and lets windows give pages back."""
        for s, n in zip(slots, new_lens):
            self.lengths[s] = n
            for g in self.paged:
                g.trim(s, n)
        for g in self.paged:
            g.upload()

    # ---- views ---------------------------------------------------------------------
    def view(self, layer: int):
        g = self._of_layer.get(layer)
        return None if g is None else g.view(layer)

    def check(self) -> None:
        """Host-side consistency: nothing lost, nothing held twice."""
        self.slots.check()
        for g in self.paged:
            g.pool.check()
            seen = set()
            for s in range(self.max_slots):
                pages = [int(p) for p in g.table_host[s] if p >= 0]
                if pages and not self.slots.is_held(s):
                    raise CacheStateError(f"free slot {s} still holds pages")
                for p in pages:
                    if p in seen:
                        raise CacheStateError(f"page {p} is in two places")
                    if not g.pool.is_held(p):
                        raise CacheStateError(f"page {p} is in a table but free")
                    seen.add(p)
            if len(seen) != g.pool.held_count:
                raise CacheStateError("a held page is in no table")

    def bytes_held(self) -> int:
        return sum(g.storage.numel() * g.storage.element_size() for g in self.paged + self.states)
