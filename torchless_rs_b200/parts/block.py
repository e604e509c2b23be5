"""The arrangement of parts in a layer.  Pre-norm residual block:
h += mixer(norm1(h)); h += feed_forward(norm2(h)); the residual is the stream before
the norm (reference: src/model/modules/layer.rs:28-56).  The stream stays in 32-bit
and each part adds into it."""
from __future__ import annotations

import torch

from .registry import register_block
from .runtime import Runtime


@register_block("prenorm")
class PreNormBlock:
    """Interface of every block: built from its four parts, `forward(x, batch)`
    updates the 32-bit stream `x` [tokens, hidden] in place."""

    def __init__(self, spec, rt: Runtime, mixer, feed_forward, mixer_norm, feed_forward_norm):
        self.rt = rt
        self.mixer = mixer
        self.feed_forward = feed_forward
        self.mixer_norm = mixer_norm
        self.feed_forward_norm = feed_forward_norm

    def forward(self, x: torch.Tensor, batch) -> None:
        xn = self.rt.workspace.get("block_normed", x.shape, self.rt.act_dtype)
        self.mixer_norm(x, xn)
        self.mixer.forward(xn, x, batch)
        self.feed_forward_norm(x, xn)
        self.feed_forward.forward(xn, x, batch)
