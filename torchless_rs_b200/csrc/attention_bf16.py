"""Tensor-core attention of the bfloat16 path, one library per head size.  `run`
returns False for a case it does not take; the caller then uses the CUDA-core
kernel."""
from __future__ import annotations

from ctypes import c_float, c_int, c_longlong
from typing import Dict

import torch

from . import build
from .ops import KernelError, _check, _need, _ptr, _stream, register_error_word

FAST_HEAD_DIMS = (32, 64, 128)
MAX_GROUP = 16        # query heads per key/value head that one instruction's rows hold
TARGET_BLOCKS = 296   # two resident blocks on each of a B200's 148 SMs: one full wave measured best
                      # (the default of `decode_splits`; the engine passes twice the device's own SM count)

for _hd in FAST_HEAD_DIMS:
    build.register_library(f"attn_bf16_hd{_hd}",
                           ("attention_decode_bf16.cu", "attention_prefill_bf16.cu") +
                           (("attention_decode_tma.cu", "attention_prefill_tc.cu") if _hd % 64 == 0 else ()),
                           (f"-DHEAD_DIM={_hd}",))
    # the same kernels with a fixed scratch array inside the library, for callers that must
    # not allocate (see attention_decode_noalloc.h); nothing in this package loads it
    build.register_library(f"attn_noalloc_bf16_hd{_hd}", ("attention_decode_noalloc.cu",),
                           (f"-DHEAD_DIM={_hd}",))


# What the split rule knows about the decode kernel (measured on a B200, head size 128, `measure attn-decode`):
BLOCK_GBS = 33.0      # one block alone streams its pages at about this rate (three pages in flight)
HBM_GBS = 6500.0      # all blocks together
MERGE_US = 2.5        # the merge kernel that more than one split needs
SPLIT_US = 0.03       # and what every further split adds to it
WAVE_US = 1.0         # set-up and the write of the partial results, once per wave of blocks


def decode_splits(batch_size: int, nkv: int, max_len: int, window, target_blocks: int = TARGET_BLOCKS,
                  head_dim: int = 128) -> int:
    """How many blocks share the keys of one (sequence, kv head): the count with the least estimated
    time, never more than there is work.  The estimate: blocks run in waves of `target_blocks`; a block
    takes its pages at BLOCK_GBS unless the wave together exceeds HBM_GBS; several splits cost a merge.
    It gives one full wave where the (sequence, kv head) pairs are few (8 sequences of 4096 tokens and 8
    kv heads: 4 splits, 24.8 us; 1 sequence: 32 splits), and where they are more than one wave it cuts
    them finer so that the last wave is not a nearly empty one (40 sequences: 4 splits 111 us, 1 split
    138 us; 20 sequences: 3 splits 57 us, 1 split 63 us; 24 or 32 sequences: 1 split)."""
    span = min(max_len, window) if window else max_len
    groups = (span + 31) // 32 + 1
    by_work = max(1, (groups + 3) // 4)          # at least one 32-key group per warp
    cap = min(by_work, 32)                       # 32: the merge kernel fetches that many splits in one round of loads
    units = max(1, batch_size * nkv)
    one_wave = max(1, min(cap, target_blocks // units))   # as many splits as fill one wave
    pages = (span + build.PAGE_TOKENS - 1) // build.PAGE_TOKENS
    page_us = build.PAGE_TOKENS * head_dim * 4 / (BLOCK_GBS * 1e3)     # keys and values, two bytes each
    together = HBM_GBS / BLOCK_GBS               # blocks that saturate the memory
    best, best_t = 1, None
    # the one-wave count against 1 to 4 splits (what was measured where the pairs exceed a wave)
    for s in sorted(set([one_wave] + [c for c in (1, 2, 3, 4) if c <= cap])):
        full, rest = divmod(units * s, target_blocks)
        waves = full * max(target_blocks / together, 1.0) + (max(rest / together, 1.0) if rest else 0.0)
        t = -(-pages // s) * page_us * waves + WAVE_US * (full + (1 if rest else 0))
        if s > 1:
            t += MERGE_US + SPLIT_US * s
        if best_t is None or t < 0.98 * best_t:      # more splits only for a gain the estimate can resolve
            best, best_t = s, t
    return best


def decode_plan(batch_size: int, nkv: int, max_len: int, window, target_blocks: int = TARGET_BLOCKS,
                head_dim: int = 128, lens=None):
    """(splits, quantum) for a decode step.  quantum 0: every sequence is cut into `splits` equal shares
    (`decode_splits`).  Where the sequences' lengths (`lens`) differ, equal shares of each sequence leave
    the longest one's blocks with most of the work; then a block takes `quantum` pages whatever the
    sequence: the long ones get more blocks that work, and `splits` is what a sequence of `max_len` (an
    upper bound of the longest) needs.  Both ways are estimated as in `decode_splits` (the longest block
    at a block's rate, all pages at the memory's rate, a further wave if more blocks work than the GPU
    holds); the quantum is taken where it is worth more than a twentieth.  Measured, 8 layers + head of
    the 7B sizes: one sequence of 32768 tokens beside seven of 1024: 1701 -> 1142 us a step."""
    n = decode_splits(batch_size, nkv, max_len, window, target_blocks, head_dim)
    if lens is None or batch_size < 2 or len(lens) != batch_size:
        return n, 0
    page = build.PAGE_TOKENS
    spans = [min(int(x), window) if window else int(x) for x in lens]
    pages = [-(-x // page) + (1 if window else 0) for x in spans]     # a window may reach into one page more
    p_long, p_total = max(pages), sum(pages)
    span_max = min(max_len, window) if window else max_len
    p_max = -(-span_max // page) + (1 if window else 0)
    page_us = page * head_dim * 4 / (BLOCK_GBS * 1e3)
    together = HBM_GBS / BLOCK_GBS

    def estimate(working: int, longest: int, splits: int) -> float:
        t = max(longest, p_total * nkv / together) * page_us
        t += (-(-working // target_blocks) - 1) * longest * page_us      # blocks beyond what the GPU holds at once
        return t + (MERGE_US + SPLIT_US * splits if splits > 1 else 0.0)

    best_t = estimate(batch_size * nkv * n, -(-p_long // n), n)
    best = (n, 0)
    for k in range(2, 33):
        quantum = -(-p_long // k)
        splits = -(-p_max // quantum)
        if splits > 32 or quantum < 2:
            break
        working = sum(-(-p // quantum) for p in pages) * nkv
        t = estimate(working, min(quantum, p_long), splits)
        if t < 0.95 * best_t:
            best_t, best = t, (splits, quantum)
    return best


class AttentionBf16:
    _by_hd: Dict[int, "AttentionBf16"] = {}

    @classmethod
    def get(cls, head_dim: int) -> "AttentionBf16":
        if head_dim not in cls._by_hd:
            cls._by_hd[head_dim] = cls(head_dim)
        return cls._by_hd[head_dim]

    def __init__(self, head_dim: int):
        self.head_dim = head_dim
        self.lib = None
        if head_dim in FAST_HEAD_DIMS:
            self.lib = build.load_library(f"attn_bf16_hd{head_dim}")
            self._decode = getattr(self.lib, f"tl_attn_decode_hd{head_dim}")
            self._decode.restype = c_int
            self._scratch = getattr(self.lib, f"tl_attn_decode_scratch_floats_hd{head_dim}")
            self._scratch.restype = c_longlong
            self._prefill = getattr(self.lib, f"tl_attn_prefill_hd{head_dim}")
            self._prefill.restype = c_int
            self._decode_tma = None
            if head_dim % 64 == 0:
                self._decode_tma = getattr(self.lib, f"tl_attn_decode_tma_hd{head_dim}")
                self._decode_tma.restype = c_int
                self._prefill_tma = getattr(self.lib, f"tl_attn_prefill_tma_hd{head_dim}")
                self._prefill_tma.restype = c_int
                self._prefill_tc = getattr(self.lib, f"tl_attn_prefill_tc_hd{head_dim}")
                self._prefill_tc.restype = c_int
                self._tc_error = getattr(self.lib, f"tl_attn_tc_take_error_hd{head_dim}")
                self._tc_error.restype = c_int
                self._tma_error = getattr(self.lib, f"tl_attn_tma_take_error_hd{head_dim}")
                self._tma_error.restype = c_int
                register_error_word(f"attn_bf16_hd{head_dim}", self.take_error)

    _targets: Dict[int, int] = {}

    @classmethod
    def _target_blocks(cls, device: torch.device) -> int:
        """Two resident blocks per SM of the device the step runs on."""
        idx = device.index if device.index is not None else torch.cuda.current_device()
        if idx not in cls._targets:
            cls._targets[idx] = 2 * torch.cuda.get_device_properties(idx).multi_processor_count
        return cls._targets[idx]

    def take_error(self) -> int:
        """Nonzero if a TMA kernel gave up on a bounded wait since the last call (synchronises)."""
        if getattr(self, "_decode_tma", None) is None:
            return 0
        return int(self._tma_error()) or int(self._tc_error())

    def decode(self, q, k_pages, v_pages, out, seq_len, seq_slot, page_table, nh, nkv, window,
               scale, n_splits, workspace, use_tma: bool = True, quantum: int = 0) -> None:
        """One new token per sequence; `q` and `out` are [sequences, nh * head_dim].  `quantum`: 0, or
        the pages a block takes (`decode_plan`; the kernel with pages by TMA only)."""
        if self.lib is None:
            raise KernelError(f"no tensor-core decode attention for head size {self.head_dim}")
        for t, n in ((q, "q"), (k_pages, "k pages"), (v_pages, "v pages"), (out, "out")):
            _need(t, torch.bfloat16, f"attn decode {n}")
        B = q.shape[0]
        floats = self._scratch(c_int(B), c_int(nh), c_int(n_splits))
        part = workspace.get("attn_decode_partials", (floats,), torch.float32)
        if self._decode_tma is not None and use_tma:
            st = self._decode_tma(_ptr(q), _ptr(k_pages), _ptr(v_pages), c_longlong(k_pages.shape[0]),
                                  _ptr(out), _ptr(part), _ptr(seq_len), _ptr(seq_slot), _ptr(page_table),
                                  c_int(page_table.stride(0)), c_int(B), c_int(nh), c_int(nkv),
                                  c_int(window or 0), c_float(scale), c_int(n_splits), c_int(quantum), _stream())
            if st != -2:
                _check(st, "attn_decode_tma")
                return
        if quantum:
            raise KernelError("attn decode: a page quantum needs the kernel with pages by TMA")
        _check(self._decode(_ptr(q), _ptr(k_pages), _ptr(v_pages), _ptr(out), _ptr(part),
                            _ptr(seq_len), _ptr(seq_slot), _ptr(page_table),
                            c_int(page_table.stride(0)), c_int(B), c_int(nh), c_int(nkv),
                            c_int(window or 0), c_float(scale), c_int(n_splits), _stream()),
               "attn_decode")

    def prefill(self, q, k_pages, v_pages, out, seq_start, seq_len, seq_slot, page_table, n_seqs,
                max_new, nh, nkv, window, scale, use_tma: bool = True, variant: str = "auto") -> None:
        """The new tokens of each sequence (packed, `seq_start` offsets) against the cache,
        which already holds their keys and values.  `variant`: "tc" = tcgen05 kernel (head
        sizes 64 and 128), "tma" = mma.sync on TMA-fed pages, "plain" = mma.sync on fragments
        from global memory, "auto" = "tc" for steps with at least 128 new tokens, else "tma"."""
        if not use_tma:
            variant = "plain"
        if variant == "auto":
            variant = "tc" if max_new >= 128 else "tma"
        if self.lib is None:
            raise KernelError(f"no tensor-core prefill attention for head size {self.head_dim}")
        for t, n in ((q, "q"), (k_pages, "k pages"), (v_pages, "v pages"), (out, "out")):
            _need(t, torch.bfloat16, f"attn prefill {n}")
        if getattr(self, "_decode_tma", None) is not None and variant == "tc":
            st = self._prefill_tc(_ptr(q), c_longlong(q.shape[0]), _ptr(k_pages), _ptr(v_pages),
                                  c_longlong(k_pages.shape[0]), _ptr(out), _ptr(seq_start), _ptr(seq_len),
                                  _ptr(seq_slot), _ptr(page_table), c_int(page_table.stride(0)),
                                  c_int(n_seqs), c_int(max_new), c_int(nh), c_int(nkv), c_int(window or 0),
                                  c_float(scale), _stream())
            if st != -2:
                _check(st, "attn_prefill_tc")
                return
            variant = "tma"
        if getattr(self, "_decode_tma", None) is not None and variant == "tma":
            st = self._prefill_tma(_ptr(q), _ptr(k_pages), _ptr(v_pages), c_longlong(k_pages.shape[0]),
                                   _ptr(out), _ptr(seq_start), _ptr(seq_len), _ptr(seq_slot),
                                   _ptr(page_table), c_int(page_table.stride(0)), c_int(n_seqs),
                                   c_int(max_new), c_int(nh), c_int(nkv), c_int(window or 0),
                                   c_float(scale), _stream())
            if st != -2:
                _check(st, "attn_prefill_tma")
                return
        _check(self._prefill(_ptr(q), _ptr(k_pages), _ptr(v_pages), _ptr(out), _ptr(seq_start),
                             _ptr(seq_len), _ptr(seq_slot), _ptr(page_table),
                             c_int(page_table.stride(0)), c_int(n_seqs), c_int(max_new), c_int(nh),
                             c_int(nkv), c_int(window or 0), c_float(scale), _stream()),
               "attn_prefill")

    def run(self, q, cache_view, out, batch, nh, nkv, window, scale, workspace) -> bool:
        if self.lib is None or nh // nkv > MAX_GROUP:
            return False
        if batch.is_decode:
            tma = getattr(self, "_decode_tma", None) is not None
            n_splits, quantum = decode_plan(batch.n_seqs, nkv, batch.len_bucket, window,
                                            self._target_blocks(q.device), self.head_dim,
                                            getattr(batch, "new_lens", None) if tma else None)
            self.decode(q, cache_view.k_pages, cache_view.v_pages, out, batch.seq_len,
                        batch.seq_slot, cache_view.page_table, nh, nkv, window, scale, n_splits,
                        workspace, quantum=quantum)
            return True
        self.prefill(q, cache_view.k_pages, cache_view.v_pages, out, batch.seq_start, batch.seq_len,
                     batch.seq_slot, cache_view.page_table, batch.n_seqs, batch.max_new, nh, nkv,
                     window, scale)
        return True
