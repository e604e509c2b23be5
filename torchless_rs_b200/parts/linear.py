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


class Matmul:
    def __init__(self, rt: Runtime):
        self.rt = rt
        self.fast = None
        if not rt.is_f32:
            from ..csrc import gemm_bf16
            self.fast = gemm_bf16.GemmBf16.get()

    def __call__(self, a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, mode: int) -> None:
        if self.fast is not None and self.fast.run(a, w, out, mode):
            return
        self.rt.ops.gemm_generic(a, w, out, mode)
