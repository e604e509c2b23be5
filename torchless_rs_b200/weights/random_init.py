"""Random weights from a configuration and a seed.

The reference has no random-weights mode of its own; its test fixture is drawn
with an unseeded normal generator (tests/generate_test_model.py:89-110).  Here
every tensor has its own generator seeded by (seed, tensor name), so a tensor's
values do not depend on which other tensors exist or in which order they are
drawn.  Matrices and tables are N(0, 0.02); norm weights are 1 + N(0, 0.1).
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Iterator, Mapping, Tuple

import torch

from .loader import TensorSpec
from .safetensors_io import write_safetensors

MATRIX_STD = 0.02
NORM_STD = 0.1


def _tensor_seed(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{seed}:{name}".encode("utf-8")).digest()
    return int.from_bytes(h[:8], "little") & 0x7FFF_FFFF_FFFF_FFFF


def random_tensor(name: str, spec: TensorSpec, seed: int, dtype: torch.dtype,
                  device: str | torch.device = "cpu") -> torch.Tensor:
    """One tensor.  Vectors (one dimension) are taken to be norm weights.  Values
    are drawn in 32-bit and then rounded to `dtype`.  CPU and CUDA generators give
    different values for the same seed."""
    dev = torch.device(device)
    g = torch.Generator(device=dev)
    g.manual_seed(_tensor_seed(seed, name))
    if spec.integer:
        return torch.randint(0, 2 ** 15, spec.shape, generator=g, device=dev, dtype=torch.int32)
    if dev.type == "cuda" and dtype == torch.bfloat16:
        t = torch.empty(spec.shape, dtype=dtype, device=dev)
        t.normal_(0.0, 1.0, generator=g)
    else:
        t = torch.randn(spec.shape, generator=g, device=dev, dtype=torch.float32)
    if len(spec.shape) == 1:
        t = t.float().mul_(NORM_STD).add_(1.0)
    else:
        t = t.mul_(MATRIX_STD)
    return t.to(dtype)


def random_tensors(expected: Mapping[str, TensorSpec], seed: int, dtype: torch.dtype,
                   device: str | torch.device = "cpu") -> Iterator[Tuple[str, torch.Tensor]]:
    for name, spec in expected.items():
        yield name, random_tensor(name, spec, seed, dtype, device)


def write_random_model(config, out_dir: str, seed: int, dtype: torch.dtype = torch.bfloat16) -> str:
    """Writes `config.json` and `model.safetensors` for `config` (a registered
    configuration object) into `out_dir` and returns the folder."""
    from ..engine.model import expected_tensors
    os.makedirs(out_dir, exist_ok=True)
    expected = expected_tensors(config.model_spec())
    d = config.to_dict()
    d["torch_dtype"] = {torch.bfloat16: "bfloat16", torch.float32: "float32",
                        torch.float16: "float16"}[dtype]
    with open(os.path.join(out_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(d, f, indent=1)
    write_safetensors(os.path.join(out_dir, "model.safetensors"),
                      list(random_tensors(expected, seed, dtype)),
                      metadata={"format": "pt", "seed": str(seed)})
    return out_dir
