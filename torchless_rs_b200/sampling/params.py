"""Sampling options, with the names and meanings of the reference's
`SamplingConfig` (src/sampler/mod.rs:17-54): temperature <= 0 is greedy; top_k
keeps the k largest scaled logits (ignored if 0 or >= vocabulary); top_p keeps the
smallest set of probabilities that sums to >= p (ignored unless 0 < p < 1)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 1.0
    top_k: Optional[int] = None
    top_p: Optional[float] = None

    @classmethod
    def greedy(cls) -> "SamplingParams":
        return cls(temperature=0.0)

    @property
    def is_greedy(self) -> bool:
        return self.temperature <= 0.0


_MASK = (1 << 64) - 1


def _mix(z: int) -> int:
    z = (z + 0x9E3779B97F4A7C15) & _MASK
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK
    return z ^ (z >> 31)


def uniform_for(seed: int, sequence: int, step: int) -> float:
    """A number in [0, 1) with 24 random bits that depends only on (seed, sequence,
    step), so a draw can be repeated anywhere.  The reference draws from an unseeded
    thread generator (src/sampler/mod.rs:226-227)."""
    h = _mix(_mix(_mix(seed & _MASK) ^ (sequence & _MASK)) ^ (step & _MASK))
    return (h >> 40) / float(1 << 24)
