"""Error types of the weights layer."""
from __future__ import annotations

from typing import List, Sequence, Tuple


class SafetensorsFormatError(ValueError):
    """The file is not a well-formed safetensors container."""


class WeightsMismatchError(ValueError):
    """The tensors in the model folder are not the tensors the model asks for.

    One error carries the whole comparison: names the model needs and the files
    lack, names the files hold and the model does not know, and tensors whose
    shape differs from what the configuration implies."""

    def __init__(self, where: str, missing: Sequence[str], unexpected: Sequence[str],
                 wrong_shape: Sequence[Tuple[str, Tuple[int, ...], Tuple[int, ...]]],
                 wrong_dtype: Sequence[Tuple[str, str]] = ()):
        self.where = where
        self.missing: List[str] = list(missing)
        self.unexpected: List[str] = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        self.wrong_dtype = list(wrong_dtype)
        lines = [f"{where}: the tensors do not match the configuration"]
        if self.missing:
            lines.append(f"  missing ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shape ({len(self.wrong_shape)}): " + ", ".join(
                f"{n} expected {list(e)} got {list(g)}" for n, e, g in self.wrong_shape))
        if self.wrong_dtype:
            lines.append(f"  unsupported dtype ({len(self.wrong_dtype)}): " + ", ".join(
                f"{n} is {d}" for n, d in self.wrong_dtype))
        super().__init__("\n".join(lines))
