"""Matrix products of the parts: picks the kernel for a shape.

`out (op)= a @ w.T` with 32-bit accumulation.  In 32-bit everything runs on the
CUDA-core kernels.  In bfloat16 the tensor-core kernels take the shapes they are
built for and the CUDA-core kernels take the rest; which kernel ran never changes
what is computed, only its rounding order.
"""
from __future__ import annotations

import torch

from ..csrc import ops
from .runtime import Runtime


class NormCarry:
    """The input of a norm that the product before it has already prepared: `xw` = the
    stream times the norm's weight (bfloat16), `ss` = partial sums of squares of each row
    of the stream, one per 128 columns.  The product after it scales its outputs by
    1/rms.  `valid` says whether the last producer filled it."""

    def __init__(self, xw: torch.Tensor, ss: torch.Tensor, size: int, eps: float):
        self.xw, self.ss, self.size, self.eps = xw, ss, size, eps
        self.tiles = ss.shape[1]
        self.valid = False


def new_carry(rt: Runtime, name: str, n_tokens: int, size: int, eps: float) -> NormCarry:
    ws = rt.workspace
    tiles = (size + 127) // 128
    return NormCarry(ws.get(f"carry_xw_{name}", (n_tokens, size), torch.bfloat16),
                     ws.get(f"carry_ss_{name}", (n_tokens, tiles), torch.float32), size, eps)


class Matmul:
    def __init__(self, rt: Runtime):
        self.rt = rt
        self.fast = None
        if not rt.is_f32:
            from ..csrc import gemm_bf16
            self.fast = gemm_bf16.GemmBf16.get()

    def __call__(self, a, w: torch.Tensor, out: torch.Tensor, mode: int, emit=None, rope=None) -> bool:
        """`a` is an activation tensor or a `NormCarry`.  `emit` = (norm weight, NormCarry)
        asks the product (mode 1) to prepare the next norm's input if it can.  `rope` (a
        `gemm_bf16.RopeArgs`) asks the q/k/v product to rotate and write q, k and v itself;
        the return value says whether it did (then `out` was not written)."""
        scaled = a if isinstance(a, NormCarry) else None
        if scaled is not None:
            if self.fast is None or not self.fast.run(scaled.xw, w, out, mode, scaled=scaled, rope=rope):
                raise ops.KernelError("a folded norm reached a product that cannot apply it")
            return self.fast.rope_applied
        if emit is not None:
            emit[1].valid = False
        if self.fast is not None and self.fast.run(a, w, out, mode, emit=emit, rope=rope):
            return self.fast.rope_applied
        self.rt.ops.gemm_generic(a, w, out, mode)
        return False
