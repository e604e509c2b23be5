"""Dense SwiGLU feed-forward: down( silu(gate x) * (up x) )
(reference: src/model/modules/mlp.rs:23-45).  Gate and up rows are stacked into one
matrix at load time so that one product yields both and the SiLU-gate happens where
the product is written."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..config.spec import PartSpec
from ..csrc import ops
from ..weights.loader import TensorSpec
from .linear import Matmul
from .registry import register_feed_forward
from .runtime import Runtime


@register_feed_forward("swiglu")
class SwiGLU:
    """Parameters: `hidden_size`, `intermediate_size`.  Interface of every
    feed-forward: `expected_tensors(spec, prefix)` (a class method), `load(weights)`, and `forward(xn, residual, batch)`,
    which adds its output to the 32-bit `residual` in place."""
    graph_safe = True   # forward launches kernels whose arguments do not depend on host values


    def __init__(self, spec: PartSpec, prefix: str, rt: Runtime):
        self.hidden = int(spec.params["hidden_size"])
        self.inter = int(spec.params["intermediate_size"])
        self.prefix = prefix
        self.rt = rt
        self.matmul = Matmul(rt)
        self.w_gate_up: Optional[torch.Tensor] = None
        self.w_down: Optional[torch.Tensor] = None

    @classmethod
    def expected_tensors(cls, spec: PartSpec, prefix: str) -> Dict[str, TensorSpec]:
        h, i = int(spec.params["hidden_size"]), int(spec.params["intermediate_size"])
        return {
            f"{prefix}.gate_proj.weight": TensorSpec((i, h)),
            f"{prefix}.up_proj.weight": TensorSpec((i, h)),
            f"{prefix}.down_proj.weight": TensorSpec((h, i)),
        }

    def load(self, weights: Dict[str, torch.Tensor]) -> None:
        p = self.prefix
        self.w_gate_up = self.rt.stack([weights[f"{p}.gate_proj.weight"], weights[f"{p}.up_proj.weight"]])
        self.w_down = self.rt.matrix(weights[f"{p}.down_proj.weight"])

    accepts_carry = True   # `xn` may be a NormCarry; `emit` may ask for the next norm's input

    def forward(self, xn, residual: torch.Tensor, batch, emit=None) -> None:
        T = residual.shape[0]
        act = self.rt.workspace.get("ffn_act", (T, self.inter), self.rt.act_dtype)
        self.matmul(xn, self.w_gate_up, act, ops.MODE_SWIGLU)
        self.matmul(act, self.w_down, residual, ops.MODE_ACCUM_F32, emit=emit)
