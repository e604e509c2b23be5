"""Python face of the CUDA launchers: argument checks, then one C call per kernel.

There is no other implementation behind these functions.  A tensor that is not on
a CUDA device, a missing library or a launch that the driver rejects raises
`KernelError`; nothing falls back to the CPU or to library model code.
"""
from __future__ import annotations

from ctypes import c_float, c_int, c_void_p
from typing import Callable, Dict, Optional

import torch

from . import build

MODE_STORE_F32 = 0
MODE_ACCUM_F32 = 1
MODE_SWIGLU = 2
MODE_STORE_ACT = 3

PAGE = build.PAGE_TOKENS  # tokens per cache page; the kernels are compiled with the same number


class KernelError(RuntimeError):
    pass


_SUFFIX = {torch.float32: "f32", torch.bfloat16: "bf16"}
_error_words: Dict[str, Callable[[], int]] = {}


def register_error_word(name: str, take: Callable[[], int]) -> None:
    """A kernel library whose waits are bounded names the function that reads and clears
    its error word (nonzero: a kernel gave up waiting, its results are not valid)."""
    _error_words[name] = take


def check_kernel_errors() -> None:
    """Reads every registered error word (this synchronises the device) and raises if one is
    set.  Callers use it where they wait for results anyway."""
    bad = {name: code for name, code in ((n, take()) for n, take in _error_words.items()) if code}
    if bad:
        raise KernelError("a kernel ran out of a bounded wait, its results are not valid: " +
                          ", ".join(f"{n}: code {c}" for n, c in bad.items()))
_counter = {"launches": 0}
_by_name: Dict[str, int] = {}


def launches() -> int:
    """Kernels launched through this module since the process started."""
    return _counter["launches"]


def launch_counts() -> Dict[str, int]:
    """The same count by launcher ("rmsnorm", "gemm_tc", "rope_cache_write", ...): what a
    test reads to see which kernels a step was made of."""
    return dict(_by_name)


def add_launches(n, sign: int = 1) -> None:
    """Counts kernels that ran without passing through this module: a replayed CUDA
    graph launches the kernels that were counted while it was recorded.  `n` is a number or
    a dictionary by launcher as `launch_counts` returns it."""
    if isinstance(n, dict):
        for k, v in n.items():
            _by_name[k] = _by_name.get(k, 0) + sign * v
        n = sum(n.values())
    _counter["launches"] += sign * n


def counts_since(before: Dict[str, int]) -> Dict[str, int]:
    """Launches by launcher since `before` (an earlier `launch_counts()`)."""
    return {k: v - before.get(k, 0) for k, v in _by_name.items() if v != before.get(k, 0)}


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> c_void_p:
    """The current stream's handle.  Asked of torch's C layer directly where it offers that: the Python
    `current_stream()` object costs some 15 us a call, a fifth of the host's time in a step launched
    kernel by kernel."""
    if _raw_stream is not None:
        return c_void_p(_raw_stream(torch.cuda.current_device()))
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(t: Optional[torch.Tensor]) -> c_void_p:
    if t is None:
        return c_void_p(0)
    if not t.is_cuda:
        raise KernelError("kernel argument is not on a CUDA device; this package has no CPU path")
    return c_void_p(t.data_ptr())


def _check(status: int, what: str) -> None:
    _counter["launches"] += 1
    _by_name[what] = _by_name.get(what, 0) + 1
    if status == 0:
        return
    if status == -1:
        raise KernelError(f"{what}: the kernel refused its arguments")
    if status == -2:
        raise KernelError(f"{what}: these sizes are not supported by this kernel")
    raise KernelError(f"{what}: CUDA error {status} at launch")


def _need(t: torch.Tensor, dtype: torch.dtype, what: str, contiguous: bool = True) -> None:
    if t.dtype != dtype:
        raise KernelError(f"{what}: expected {dtype}, got {t.dtype}")
    if contiguous and not t.is_contiguous():
        raise KernelError(f"{what}: tensor must be contiguous")


class CoreOps:
    """The kernels of one activation type (float32 or bfloat16)."""

    def __init__(self, act_dtype: torch.dtype):
        if act_dtype not in _SUFFIX:
            raise KernelError(f"no kernels for activation type {act_dtype}")
        self.act_dtype = act_dtype
        self.suffix = _SUFFIX[act_dtype]
        self.lib = build.load_library(f"core_{self.suffix}")
        for base in ("tl_embed", "tl_softcap", "tl_advance_step", "tl_regroup_step", "tl_convert", "tl_rmsnorm", "tl_rope_cache_write", "tl_silu_mul",
                     "tl_gemm_generic", "tl_attn_generic"):
            fn = getattr(self.lib, f"{base}_{self.suffix}")
            fn.restype = c_int
            setattr(self, "_" + base, fn)

    # x[t, :] = table[tokens[t], :]
    def embed(self, tokens: torch.Tensor, table: torch.Tensor, x: torch.Tensor,
              token_from: Optional[torch.Tensor] = None,
              token_src: Optional[torch.Tensor] = None, scale: float = 1.0,
              position_table: Optional[torch.Tensor] = None,
              token_pos: Optional[torch.Tensor] = None) -> None:
        """x[t] = scale * table[token t] (+ position_table[token_pos[t]]).  With `token_src`
        (int32 on the device), token t is token_src[token_from[t]] wherever token_from[t] >= 0,
        else tokens[t]."""
        _need(tokens, torch.int32, "embed tokens")
        _need(table, self.act_dtype, "embed table")
        _need(x, torch.float32, "embed out")
        if token_src is not None:
            _need(token_src, torch.int32, "embed token source")
            _need(token_from, torch.int32, "embed token index")
        T, H = x.shape
        max_pos = 0
        if position_table is not None:
            _need(position_table, self.act_dtype, "embed position table")
            _need(token_pos, torch.int32, "embed token positions")
            if position_table.shape[1] != H:
                raise KernelError("embed: the position table's width is not the stream's")
            max_pos = position_table.shape[0]
        _check(self._tl_embed(_ptr(tokens), _ptr(token_from if token_src is not None else None),
                              _ptr(token_src), _ptr(table), _ptr(x), c_int(T), c_int(H),
                              c_int(table.shape[0]), c_float(scale), _ptr(position_table),
                              _ptr(token_pos if position_table is not None else None), c_int(max_pos),
                              _stream()), "embed")

    def convert_into(self, src: torch.Tensor, dst: torch.Tensor) -> None:
        """dst (activation type, contiguous, on the device) = src (32-bit, bfloat16 or float16, the
        same number of elements, contiguous, on the device): a weight on its way into the model."""
        kinds = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}
        if src.dtype not in kinds:
            raise KernelError(f"convert: unsupported stored type {src.dtype}")
        _need(dst, self.act_dtype, "convert destination")
        if not src.is_contiguous() or src.numel() != dst.numel():
            raise KernelError("convert: source and destination must be contiguous and of one size")
        from ctypes import c_longlong
        _check(self._tl_convert(_ptr(src), c_int(kinds[src.dtype]), _ptr(dst), c_longlong(dst.numel()), _stream()),
               "convert")

    def advance_step(self, token_pos: torch.Tensor, seq_len: torch.Tensor) -> None:
        """Every row's position and length go up by one, on the device (a decode step of the same
        batch as the step before)."""
        _need(token_pos, torch.int32, "advance positions")
        _need(seq_len, torch.int32, "advance lengths")
        if token_pos.numel() != seq_len.numel():
            raise KernelError("advance_step: one position and one length per row are needed")
        _check(self._tl_advance_step(_ptr(token_pos), _ptr(seq_len), c_int(seq_len.numel()), _stream()),
               "advance_step")

    REGROUP_MAX_ROWS = 256

    def regroup_step(self, old_pos: torch.Tensor, old_len: torch.Tensor, old_slot: torch.Tensor,
                     base: torch.Tensor, offsets, keep, token_from) -> None:
        """The arrays of a decode step of the rows `keep` of the decode step before (whose positions,
        lengths and slots are `old_*`), written into `base` at `offsets` (eight starts, in the order
        tokens, token_seq, token_pos, seq_slot, seq_start, seq_len, want_rows, token_from); row j takes
        its token from place token_from[j] of the sampler's output.  The old arrays may lie in `base`."""
        from ctypes import c_ushort
        n = len(keep)
        if n > self.REGROUP_MAX_ROWS or len(token_from) != n or len(offsets) != 8:
            raise KernelError("regroup_step: at most 256 rows, one source place per row, eight offsets")
        if n and (max(keep) >= old_pos.numel() or max(keep) > 65535 or max(token_from) > 65535
                  or min(keep) < 0 or min(token_from) < 0):
            raise KernelError("regroup_step: a row or a source place is out of range")
        for t, what in ((old_pos, "positions"), (old_len, "lengths"), (old_slot, "slots"), (base, "buffer")):
            _need(t, torch.int32, "regroup " + what)
        if max(offsets) + n + 1 > base.numel():
            raise KernelError("regroup_step: the new layout does not fit the buffer")
        _check(self._tl_regroup_step(_ptr(old_pos), _ptr(old_len), _ptr(old_slot), _ptr(base),
                                     (c_int * 8)(*[int(o) for o in offsets]), c_int(n),
                                     (c_ushort * max(n, 1))(*[int(k) for k in keep]),
                                     (c_ushort * max(n, 1))(*[int(f) for f in token_from]), _stream()),
               "regroup_step")

    def softcap(self, logits: torch.Tensor, cap: float) -> None:
        """logits <- cap * tanh(logits / cap), in place."""
        _need(logits, torch.float32, "softcap logits")
        from ctypes import c_longlong
        _check(self._tl_softcap(_ptr(logits), c_longlong(logits.numel()), c_float(cap), _stream()),
               "softcap")

    def rmsnorm(self, x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor,
                rows: Optional[torch.Tensor] = None) -> None:
        _need(x, torch.float32, "rmsnorm in")
        _need(out, self.act_dtype, "rmsnorm out")
        if weight.dtype not in (torch.float32, torch.bfloat16):
            raise KernelError(f"rmsnorm weight: unsupported dtype {weight.dtype}")
        n_rows, H = out.shape
        if weight.numel() != H or x.shape[1] != H:
            raise KernelError("rmsnorm: sizes do not match")
        if rows is not None:
            _need(rows, torch.int32, "rmsnorm rows")
        _check(self._tl_rmsnorm(_ptr(x), _ptr(rows), _ptr(weight),
                                c_int(1 if weight.dtype == torch.float32 else 0), _ptr(out),
                                c_int(n_rows), c_int(H), c_float(eps), _stream()), "rmsnorm")

    def rope_cache_write(self, qkv: torch.Tensor, q_out: torch.Tensor,
                         k_pages: Optional[torch.Tensor], v_pages: Optional[torch.Tensor],
                         token_pos: torch.Tensor, token_seq: torch.Tensor, seq_slot: torch.Tensor,
                         page_table: Optional[torch.Tensor], inv_freq: Optional[torch.Tensor],
                         style: int, nh: int, nkv: int, hd: int) -> None:
        _need(qkv, torch.float32, "rope qkv")
        _need(q_out, self.act_dtype, "rope q out")
        T = qkv.shape[0]
        stride = 0
        if k_pages is not None:
            _need(k_pages, self.act_dtype, "k pages")
            _need(v_pages, self.act_dtype, "v pages")
            _need(page_table, torch.int32, "page table")
            stride = page_table.stride(0)
            if qkv.shape[1] < (nh + 2 * nkv) * hd:
                raise KernelError("rope: qkv has too few columns")
        if inv_freq is not None:
            _need(inv_freq, torch.float32, "inv_freq")
            if inv_freq.numel() != hd // 2:
                raise KernelError("rope: inv_freq must have head_dim/2 entries")
        _check(self._tl_rope_cache_write(
            _ptr(qkv), c_int(qkv.stride(0)), _ptr(q_out), _ptr(k_pages), _ptr(v_pages),
            _ptr(token_pos), _ptr(token_seq), _ptr(seq_slot), _ptr(page_table), c_int(stride),
            _ptr(inv_freq), c_int(style), c_int(T), c_int(nh), c_int(nkv), c_int(hd), _stream()),
            "rope_cache_write")

    def silu_mul(self, gu: torch.Tensor, out: torch.Tensor) -> None:
        _need(gu, torch.float32, "silu_mul in")
        _need(out, self.act_dtype, "silu_mul out")
        T, I = out.shape
        _check(self._tl_silu_mul(_ptr(gu), _ptr(out), c_int(T), c_int(I), _stream()), "silu_mul")

    def gemm_generic(self, a: torch.Tensor, w: torch.Tensor, c: torch.Tensor, mode: int) -> None:
        """c (op)= a @ w.T; in SwiGLU mode w holds the gate rows, then the up rows."""
        _need(a, self.act_dtype, "gemm a", contiguous=False)
        _need(w, self.act_dtype, "gemm w", contiguous=False)
        want_c = torch.float32 if mode in (MODE_STORE_F32, MODE_ACCUM_F32) else self.act_dtype
        _need(c, want_c, "gemm c", contiguous=False)
        M, K = a.shape
        N = c.shape[1]
        rows_w = 2 * N if mode == MODE_SWIGLU else N
        if w.shape != (rows_w, K) or c.shape[0] != M:
            raise KernelError(f"gemm: shapes do not fit: a {tuple(a.shape)} w {tuple(w.shape)} "
                              f"c {tuple(c.shape)} mode {mode}")
        if a.stride(1) != 1 or w.stride(1) != 1 or c.stride(1) != 1:
            raise KernelError("gemm: the last dimension must be contiguous")
        _check(self._tl_gemm_generic(_ptr(a), c_int(a.stride(0)), _ptr(w), c_int(w.stride(0)),
                                     _ptr(c), c_int(c.stride(0)), c_int(M), c_int(N), c_int(K),
                                     c_int(mode), _stream()), "gemm_generic")

    def attn_generic(self, q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
                     out: torch.Tensor, token_pos: torch.Tensor, token_seq: torch.Tensor,
                     seq_slot: torch.Tensor, page_table: torch.Tensor, nh: int, nkv: int, hd: int,
                     window: Optional[int], scale: float) -> None:
        for t, n in ((q, "attn q"), (k_pages, "k pages"), (v_pages, "v pages"), (out, "attn out")):
            _need(t, self.act_dtype, n)
        _need(page_table, torch.int32, "page table")
        T = q.shape[0]
        _check(self._tl_attn_generic(
            _ptr(q), _ptr(k_pages), _ptr(v_pages), _ptr(out), _ptr(token_pos), _ptr(token_seq),
            _ptr(seq_slot), _ptr(page_table), c_int(page_table.stride(0)), c_int(T), c_int(nh),
            c_int(nkv), c_int(hd), c_int(window or 0), c_float(scale), _stream()), "attn_generic")


class SamplingOps:
    def __init__(self):
        self.lib = build.load_library("sampling")
        self.lib.tl_argmax.restype = c_int
        self.lib.tl_sample.restype = c_int

    def argmax(self, logits: torch.Tensor, out: torch.Tensor) -> None:
        _need(logits, torch.float32, "argmax logits", contiguous=False)
        _need(out, torch.int32, "argmax out")
        rows, V = logits.shape
        if logits.stride(1) != 1:
            raise KernelError("argmax: the last dimension must be contiguous")
        _check(self.lib.tl_argmax(_ptr(logits), c_int(logits.stride(0)), c_int(rows), c_int(V),
                                  _ptr(out), _stream()), "argmax")

    def sample(self, logits: torch.Tensor, temperature: float, top_k: int, top_p: float,
               uniform: torch.Tensor, out: torch.Tensor) -> None:
        _need(logits, torch.float32, "sample logits", contiguous=False)
        _need(uniform, torch.float32, "sample uniform")
        _need(out, torch.int32, "sample out")
        rows, V = logits.shape
        if logits.stride(1) != 1 or uniform.numel() < rows or out.numel() < rows:
            raise KernelError("sample: bad arguments")
        _check(self.lib.tl_sample(_ptr(logits), c_int(logits.stride(0)), c_int(rows), c_int(V),
                                  c_float(temperature), c_int(top_k), c_float(top_p),
                                  _ptr(uniform), _ptr(out), _stream()), "sample")


_core: dict = {}
_sampling: list = []


def core_ops(act_dtype: torch.dtype) -> CoreOps:
    if act_dtype not in _core:
        _core[act_dtype] = CoreOps(act_dtype)
    return _core[act_dtype]


def sampling_ops() -> SamplingOps:
    if not _sampling:
        _sampling.append(SamplingOps())
    return _sampling[0]
