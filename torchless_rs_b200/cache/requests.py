"""What a mixer asks of the cache.  A mixer names its need; the cache groups
layers with equal needs and gives each group storage of its own."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch


@dataclass(frozen=True)
class PagedKVRequest:
    """Keys and values of every position (window None), or of the last `window`
    positions only."""
    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class StateRequest:
    """Per-sequence state of fixed size, zero when a sequence starts."""
    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32
