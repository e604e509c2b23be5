"""Rotary position encoding with half-split pairing: dimension i turns with
dimension i + head_dim/2 by the angle pos * theta^(-i / (head_dim/2))
(reference: src/kernels/mod.rs:572-608).  The part owns the table of inverse
frequencies and names the pairing; the mixer's kernel applies the rotation where
it reads q and k, with angle, sine and cosine in 32-bit."""
from __future__ import annotations

import torch

from ..config.spec import PartSpec
from .registry import register_position
from .runtime import Runtime

STYLE_HALF_SPLIT = 0
STYLE_INTERLEAVED = 1


@register_position("rope_half_split")
class RotaryHalfSplit:
    """Parameters: `head_dim`, `theta`.  Interface of every rotary position part:
    `inv_freq` ([head_dim/2] float32 on the device) and `style`."""
    style = STYLE_HALF_SPLIT

    def __init__(self, spec: PartSpec, rt: Runtime):
        self.head_dim = int(spec.params["head_dim"])
        self.theta = float(spec.params["theta"])
        half = self.head_dim // 2
        i = torch.arange(half, dtype=torch.float64)
        inv = 1.0 / torch.pow(torch.tensor(self.theta, dtype=torch.float64), i / half)
        self.inv_freq = inv.to(torch.float32).to(rt.device)
