"""Tensor-core attention of the bfloat16 path, one library per head size.  `run`
returns False for a case it does not take; the caller then uses the CUDA-core
kernel."""
from __future__ import annotations

from typing import Dict


class AttentionBf16:
    _by_hd: Dict[int, "AttentionBf16"] = {}

    @classmethod
    def get(cls, head_dim: int) -> "AttentionBf16":
        if head_dim not in cls._by_hd:
            cls._by_hd[head_dim] = cls(head_dim)
        return cls._by_hd[head_dim]

    def __init__(self, head_dim: int):
        self.head_dim = head_dim

    def run(self, q, cache_view, out, batch, nh, nkv, window, scale, workspace) -> bool:
        return False
