"""Weights of a model folder, looked up by tensor name and checked against what
the model asks for.

The reference asks for its tensors one by one and stops at the first that is
absent ("Tensor '{}' not found", src/loader/parameters.rs:913); here the whole
folder is compared with the model's list first and one error reports every
difference.  A folder holds `model.safetensors`, or
`model.safetensors.index.json` with its shards (the reference's sharded reader
only merges names, src/loader/formats/safetensors.rs:283-318).

Storage rule: bfloat16 tensors are kept in bfloat16, integer tensors become
int32, and a tensor stored in 32-bit floating point stays in 32 bits.  A float16
tensor becomes bfloat16 (rounded to nearest even) for a model that runs in
bfloat16 and is widened exactly to 32 bits for a model that runs in 32-bit, as
the reference widens it (src/loader/formats/safetensors.rs:374-380), so that the
32-bit path computes with the stored values.  What a part then computes with is
the part's own decision.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Dict, Mapping, Tuple

import torch

from .errors import SafetensorsFormatError, WeightsMismatchError
from .safetensors_io import SafetensorsFile

_FLOATS = (torch.float64, torch.float32, torch.float16, torch.bfloat16)
_INTS = (torch.int64, torch.int32, torch.int16, torch.int8, torch.uint8, torch.bool)


@dataclass(frozen=True)
class TensorSpec:
    """What a part expects of one tensor: its exact shape, and whether it is a
    table of integers."""
    shape: Tuple[int, ...]
    integer: bool = False


def storage_dtype(stored: torch.dtype, run_dtype: torch.dtype = torch.bfloat16) -> torch.dtype:
    """The type a stored tensor is kept in by a model that runs in `run_dtype`."""
    if stored in (torch.float32, torch.float64):
        return torch.float32
    if stored == torch.bfloat16:
        return torch.bfloat16
    if stored == torch.float16:
        return torch.float32 if run_dtype == torch.float32 else torch.bfloat16
    if stored in _INTS:
        return torch.int32
    raise TypeError(f"unsupported stored dtype {stored}")


class WeightSource:
    """Name -> tensor over the files of one model folder."""

    def __init__(self, model_dir: str, run_dtype: torch.dtype = torch.bfloat16):
        self.model_dir = model_dir
        self.run_dtype = run_dtype
        self.files = []
        self.where: Dict[str, SafetensorsFile] = {}
        single = os.path.join(model_dir, "model.safetensors")
        index = os.path.join(model_dir, "model.safetensors.index.json")
        if os.path.isfile(index):
            with open(index, "r", encoding="utf-8") as f:
                try:
                    weight_map = json.load(f)["weight_map"]
                except (json.JSONDecodeError, KeyError, TypeError) as e:
                    raise SafetensorsFormatError(f"{index}: no usable 'weight_map' ({e})") from e
            opened: Dict[str, SafetensorsFile] = {}
            for name, shard in weight_map.items():
                if shard not in opened:
                    p = os.path.join(model_dir, shard)
                    if not os.path.isfile(p):
                        raise SafetensorsFormatError(f"{index}: shard '{shard}' is missing")
                    opened[shard] = SafetensorsFile(p)
                    self.files.append(opened[shard])
            for sf in self.files:
                for name in sf.names():
                    if name in self.where:
                        raise SafetensorsFormatError(
                            f"{model_dir}: tensor '{name}' is in two shards")
                    self.where[name] = sf
        elif os.path.isfile(single):
            sf = SafetensorsFile(single)
            self.files.append(sf)
            self.where = {n: sf for n in sf.names()}
        else:
            raise FileNotFoundError(
                f"{model_dir}: neither model.safetensors nor model.safetensors.index.json found")

    def names(self):
        return list(self.where)

    def shape(self, name: str) -> Tuple[int, ...]:
        return self.where[name].shape(name)

    def stored_dtype(self, name: str) -> torch.dtype:
        return self.where[name].dtype(name)

    def tensor(self, name: str) -> torch.Tensor:
        """The tensor in its storage dtype (see the module text), on the CPU."""
        t = self.where[name].tensor(name)
        want = storage_dtype(t.dtype, self.run_dtype)
        return t if t.dtype == want else t.to(want)

    def close(self) -> None:
        for f in self.files:
            f.close()


def check_against(source_name: str, have: Mapping[str, Tuple[Tuple[int, ...], torch.dtype]],
                  expected: Mapping[str, TensorSpec]) -> None:
    """Raises one `WeightsMismatchError` that lists every difference."""
    missing = sorted(n for n in expected if n not in have)
    unexpected = sorted(n for n in have if n not in expected)
    wrong_shape, wrong_dtype = [], []
    for n, spec in expected.items():
        if n not in have:
            continue
        shape, dt = have[n]
        if tuple(shape) != tuple(spec.shape):
            wrong_shape.append((n, tuple(spec.shape), tuple(shape)))
        if spec.integer != (dt in _INTS):
            wrong_dtype.append((n, str(dt).replace("torch.", "")))
    if missing or unexpected or wrong_shape or wrong_dtype:
        raise WeightsMismatchError(source_name, missing, unexpected, wrong_shape, wrong_dtype)


def load_checked(model_dir: str, expected: Mapping[str, TensorSpec],
                 run_dtype: torch.dtype = torch.bfloat16) -> Tuple[Dict[str, torch.Tensor], WeightSource]:
    """All expected tensors of the folder, by name, in their storage dtype for a model
    that runs in `run_dtype`, on the CPU.  Tensors may view the mapped files: keep the
    returned source open until they have been copied to the device."""
    src = WeightSource(model_dir, run_dtype)
    have = {n: (src.shape(n), src.stored_dtype(n)) for n in src.names()}
    check_against(model_dir, have, expected)
    return {n: src.tensor(n) for n in expected}, src
