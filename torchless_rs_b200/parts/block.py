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
    """Interface of every block: a class attribute `norm_roles` (the norms this kind of block
    takes; a layer's spec must give exactly these), a constructor `(spec, rt, mixer,
    feed_forward, norms)` with `norms` a dictionary by role, the attributes `mixer`,
    `feed_forward` and `norms`, and `forward(x, batch)`, which updates the 32-bit stream `x`
    [tokens, hidden] in place.

    Optional, for blocks that let the products around a norm take it over: `takes_carry =
    True`, `first_norm` (the norm whose input the block before may prepare; None if its mixer
    cannot use one) and `forward(x, batch, carry, next_norm)` returning a carry for
    `next_norm` or None.  A block without `takes_carry` is called with `(x, batch)` only."""
    norm_roles = ("mixer_norm", "feed_forward_norm")
    takes_carry = True

    def __init__(self, spec, rt: Runtime, mixer, feed_forward, norms):
        self.rt = rt
        self.mixer = mixer
        self.feed_forward = feed_forward
        self.norms = dict(norms)
        self.mixer_norm = norms["mixer_norm"]
        self.feed_forward_norm = norms["feed_forward_norm"]

    @property
    def first_norm(self):
        return self.mixer_norm if getattr(self.mixer, "accepts_carry", False) else None

    def forward(self, x: torch.Tensor, batch, carry=None, next_norm=None):
        """`carry`: the input of this block's first norm if the product before it prepared
        it (else None).  `next_norm`: the norm that follows this block; the block returns
        a carry for it if its last product could prepare one (else None).

        A norm is folded into its neighbours only if it says it is `foldable` and both
        neighbours say they `accepts_carry`; otherwise the norm kernel runs."""
        from .linear import new_carry
        rt = self.rt
        xn = rt.workspace.get("block_normed", x.shape, rt.act_dtype)
        fold = not rt.is_f32

        def can_fold(norm, producer, consumer):
            return (fold and norm is not None and getattr(norm, "foldable", False)
                    and getattr(producer, "accepts_carry", False)
                    and getattr(consumer, "accepts_carry", False))

        inp = carry if (carry is not None and carry.valid) else self.mixer_norm(x, xn)
        c2 = None
        if can_fold(self.feed_forward_norm, self.mixer, self.feed_forward):
            c2 = new_carry(rt, "a", x.shape[0], self.feed_forward_norm.size, self.feed_forward_norm.eps)
            self.mixer.forward(inp, x, batch, emit=(self.feed_forward_norm.weight, c2))
        else:
            self.mixer.forward(inp, x, batch)
        inp2 = c2 if (c2 is not None and c2.valid) else self.feed_forward_norm(x, xn)
        c3 = None
        if next_norm is not None and getattr(next_norm, "foldable", False) and fold and \
                getattr(self.feed_forward, "accepts_carry", False):
            c3 = new_carry(rt, "b", x.shape[0], next_norm.size, next_norm.eps)
            self.feed_forward.forward(inp2, x, batch, emit=(next_norm.weight, c3))
        else:
            self.feed_forward.forward(inp2, x, batch)
        return c3 if (c3 is not None and c3.valid) else None
