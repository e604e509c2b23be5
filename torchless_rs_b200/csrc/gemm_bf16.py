"""Tensor-core matrix products of the bfloat16 path (kernels in gemm_tc.cu).  `run`
returns False for a shape it does not take; the caller then uses the CUDA-core kernel."""
from __future__ import annotations

import ctypes
from ctypes import byref, c_float, c_int, c_void_p

import torch

from . import build
from .ops import KernelError, _check, _ptr, _stream, register_error_word

build.register_library("gemm_tc", ("gemm_tc.cu",), ())


class RopeArgs(ctypes.Structure):
    """Mirror of TlRopeArgs in gemm_tc.cu: what the q/k/v product needs to rotate q and k and
    write k and v into the cache pages itself."""
    _fields_ = [("q_out", c_void_p), ("k_pages", c_void_p), ("v_pages", c_void_p),
                ("token_pos", c_void_p), ("token_seq", c_void_p), ("seq_slot", c_void_p),
                ("page_table", c_void_p), ("inv_freq", c_void_p),
                ("table_stride", c_int), ("style", c_int), ("nh", c_int), ("nkv", c_int), ("hd", c_int)]


class GemmBf16:
    _inst = None

    @classmethod
    def get(cls) -> "GemmBf16":
        if cls._inst is None:
            cls._inst = cls()
        return cls._inst

    def __init__(self):
        self.lib = build.load_library("gemm_tc")
        self.lib.tl_gemm_tc.restype = c_int
        # declared once, so that a call passes plain numbers (no ctypes object per argument)
        P, I = c_void_p, c_int
        self.lib.tl_gemm_tc.argtypes = [P, I, P, I, P, I, I, I, I, I, I, P, I, I, c_float, P, P, I, P,
                                        ctypes.POINTER(c_int), P, ctypes.POINTER(c_int), P]
        self.lib.tl_gemm_tc_take_error.restype = c_int
        register_error_word("gemm_tc", self.take_error)
        self._scratch = {}

    def _scratch_for(self, device: torch.device):
        key = (device.type, device.index if device.index is not None else torch.cuda.current_device())
        if key not in self._scratch:
            self._scratch[key] = torch.cuda.get_device_properties(device).multi_processor_count
        return self._scratch[key]

    def run(self, a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, mode: int,
            scaled=None, emit=None, rope: "RopeArgs" = None) -> bool:
        """out (op)= a @ w.T.  Returns False for shapes this kernel does not take.

        `scaled`: a `NormCarry` whose `xw` is `a`; outputs are scaled by each row's
        1/rms from its partial sums.  `emit`: (norm weight, NormCarry) for mode 1: if the
        kernel can, it fills the carry with the next norm's input and sets `carry.valid`.
        `rope`: for the q/k/v product (mode 0): if the kernel can, it rotates and writes q, k
        and v itself instead of `out`; `self.rope_applied` says whether it did."""
        self.rope_applied = False
        if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
            return False
        if a.stride(1) != 1 or w.stride(1) != 1 or out.stride(1) != 1:
            return False
        M, K = a.shape
        N = out.shape[1]
        want = torch.float32 if mode in (0, 1) else torch.bfloat16
        if out.dtype != want or w.shape != ((2 * N if mode == 2 else N), K) or out.shape[0] != M:
            raise KernelError(f"gemm: shapes or types do not fit: a {tuple(a.shape)} w {tuple(w.shape)} "
                              f"out {tuple(out.shape)} {out.dtype} mode {mode}")
        sms = self._scratch_for(a.device)
        emitted = c_int(0)
        applied = c_int(0)
        ss_in = scaled.ss if scaled is not None else None
        nw, carry = emit if emit is not None else (None, None)
        for t in (a, w, out):
            if not t.is_cuda:
                raise KernelError("kernel argument is not on a CUDA device; this package has no CPU path")
        addr = lambda t: t.data_ptr() if t is not None else None
        st = self.lib.tl_gemm_tc(
            a.data_ptr(), a.stride(0), w.data_ptr(), w.stride(0), out.data_ptr(), out.stride(0), M, N, K, mode, sms,
            addr(ss_in), scaled.tiles if scaled is not None else 0, scaled.size if scaled is not None else 0,
            scaled.eps if scaled is not None else 0.0,
            addr(carry.xw if carry is not None else None), addr(nw),
            1 if (nw is not None and nw.dtype == torch.float32) else 0,
            addr(carry.ss if carry is not None else None), byref(emitted),
            ctypes.cast(byref(rope), c_void_p) if rope is not None else None, byref(applied), _stream())
        if st == -2:
            return False
        _check(st, "gemm_tc")
        if carry is not None:
            carry.valid = bool(emitted.value)
        self.rope_applied = bool(applied.value)
        return True

    def take_error(self) -> int:
        """Nonzero if a kernel gave up on a bounded wait since the last call (synchronises)."""
        return int(self.lib.tl_gemm_tc_take_error())
