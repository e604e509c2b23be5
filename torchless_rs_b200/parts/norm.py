"""RMSNorm: y = x / sqrt(mean(x^2) + eps) * w, computed in 32-bit
(reference: src/kernels/mod.rs:558-568, src/model/modules/rmsnorm.rs:6-25)."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..config.spec import PartSpec
from ..weights.loader import TensorSpec
from .registry import register_norm
from .runtime import Runtime


@register_norm("rmsnorm")
class RMSNorm:
    """Parameters: `size`, `eps`.  Interface of every norm: `expected_tensors(spec, prefix)` (a class method),
    `load(weights)`, and `__call__(x, out, rows=None)` from the 32-bit stream to an
    activation tensor; `rows` (int32, on the device) picks input rows."""

    foldable = True   # x / rms * w with a plain weight: the products around it can take it over

    def __init__(self, spec: PartSpec, prefix: str, rt: Runtime):
        self.size = int(spec.params["size"])
        self.eps = float(spec.params["eps"])
        self.name = f"{prefix}.weight"
        self.rt = rt
        self.weight: Optional[torch.Tensor] = None

    @classmethod
    def expected_tensors(cls, spec: PartSpec, prefix: str) -> Dict[str, TensorSpec]:
        return {f"{prefix}.weight": TensorSpec((int(spec.params["size"]),))}

    def load(self, weights: Dict[str, torch.Tensor]) -> None:
        self.weight = self.rt.vector(weights[self.name])

    def __call__(self, x: torch.Tensor, out: torch.Tensor, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        self.rt.ops.rmsnorm(x, self.weight, self.eps, out, rows)
        return out
