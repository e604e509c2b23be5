"""Random weights from a configuration and a seed.

The reference has no random-weights mode of its own; its test fixture is drawn
with an unseeded normal generator (tests/generate_test_model.py:89-110).  Here
element i of a tensor is a function of (seed, tensor name, i) alone: a
counter-based generator.  A tensor's values do not depend on which other tensors
exist, in which order they are drawn, or where: the host code below (numpy) and
the kernel in csrc/random_init.cu follow the same sequence of correctly rounded
operations and give the same bits, so a model drawn on the device can be drawn
again on the host from its seed.  Matrices and tables are N(0, 0.02); norm
weights are 1 + N(0, 0.1).

The normal numbers are Box-Muller pairs: 64 bits per pair from a mixing function
of the counter (the finaliser of splitmix64), u1 = (high 32 bits + 1) / 2^32,
angle = 2 pi (low 32 bits) / 2^32, z = sqrt(-2 ln u1) (cos, sin)(angle), with ln,
sin and cos as fixed polynomials in double precision (no library function whose
rounding could differ between machines).
"""
from __future__ import annotations

import ctypes
import hashlib
import json
import math
import os
from typing import Iterator, Mapping, Tuple

import numpy as np
import torch

from .loader import TensorSpec
from .safetensors_io import write_safetensors

MATRIX_STD = 0.02
NORM_STD = 0.1
INT_MODULUS = 2 ** 15

_GAMMA = np.uint64(0x9E3779B97F4A7C15)
_M1 = np.uint64(0xBF58476D1CE4E5B9)
_M2 = np.uint64(0x94D049BB133111EB)
_LN2 = math.log(2.0)
_HALF_PI = math.pi / 2.0
_SQRT_HALF = math.sqrt(0.5)
_LN_C = [1.0 / (2 * j + 1) for j in range(12)]
_SIN_C = [(-1.0) ** j / float(math.factorial(2 * j + 1)) for j in range(11)]
_COS_C = [(-1.0) ** j / float(math.factorial(2 * j)) for j in range(12)]
_CHUNK = 1 << 20


class _Consts(ctypes.Structure):
    """Mirror of RandomConsts in csrc/random_init.cu: the kernel computes with the host's constants."""
    _fields_ = [("ln2", ctypes.c_double), ("half_pi", ctypes.c_double), ("sqrt_half", ctypes.c_double),
                ("ln_c", ctypes.c_double * 12), ("sin_c", ctypes.c_double * 11), ("cos_c", ctypes.c_double * 12)]


def _consts() -> _Consts:
    return _Consts(_LN2, _HALF_PI, _SQRT_HALF, (ctypes.c_double * 12)(*_LN_C),
                   (ctypes.c_double * 11)(*_SIN_C), (ctypes.c_double * 12)(*_COS_C))


def tensor_key(seed: int, name: str) -> int:
    """The 64-bit key of a tensor: the first eight bytes of sha256("<seed>:<name>")."""
    h = hashlib.sha256(f"{seed}:{name}".encode("utf-8")).digest()
    return int.from_bytes(h[:8], "little")


def _mix(z: np.ndarray) -> np.ndarray:
    z = (z ^ (z >> np.uint64(30))) * _M1
    z = (z ^ (z >> np.uint64(27))) * _M2
    return z ^ (z >> np.uint64(31))


def _bits(key: int, counters: np.ndarray) -> np.ndarray:
    with np.errstate(over="ignore"):
        return _mix(np.uint64(key) + (counters + np.uint64(1)) * _GAMMA)


def standard_normals(key: int, start: int, count: int) -> np.ndarray:
    """Elements start .. start + count - 1 of the stream of `key`, as float64.  Every line is
    one correctly rounded operation per element, in the order the kernel uses."""
    i = np.arange(start, start + count, dtype=np.uint64)
    bits = _bits(key, i >> np.uint64(1))
    k1 = (bits >> np.uint64(32)).astype(np.float64)
    k2 = (bits & np.uint64(0xFFFFFFFF)).astype(np.float64)
    u1 = (k1 + 1.0) * (1.0 / 4294967296.0)
    m, e = np.frexp(u1)
    low = m < _SQRT_HALF
    m = np.where(low, m * 2.0, m)
    e = (e - low).astype(np.float64)
    s = (m - 1.0) / (m + 1.0)
    s2 = s * s
    p = np.full_like(s, _LN_C[11])
    for j in range(10, -1, -1):
        p = p * s2 + _LN_C[j]
    ln_u = e * _LN2 + (2.0 * s) * p
    r = np.sqrt(-2.0 * ln_u)
    t4 = k2 * (1.0 / 1073741824.0)
    q = np.floor(t4)
    x = (t4 - q) * _HALF_PI
    x2 = x * x
    sp = np.full_like(x, _SIN_C[10])
    for j in range(9, -1, -1):
        sp = sp * x2 + _SIN_C[j]
    cp = np.full_like(x, _COS_C[11])
    for j in range(10, -1, -1):
        cp = cp * x2 + _COS_C[j]
    sn, cs = x * sp, cp
    q = q.astype(np.int64)
    odd_q = (q & 1) == 1
    even_i = (i & np.uint64(1)) == 0
    c = np.where(even_i, np.where(odd_q, sn, cs), np.where(odd_q, cs, sn))
    neg = np.where(even_i, (q == 1) | (q == 2), q >= 2)
    return r * (np.where(neg, -1.0, 1.0) * c)


def _host_tensor(key: int, spec: TensorSpec, scale: float, shift: float, dtype: torch.dtype) -> torch.Tensor:
    n = 1
    for d in spec.shape:
        n *= int(d)
    if spec.integer:
        i = np.arange(n, dtype=np.uint64)
        v = ((_bits(key, i) >> np.uint64(32)) % np.uint64(INT_MODULUS)).astype(np.int32)
        return torch.from_numpy(v).view(*spec.shape)
    out = torch.empty(n, dtype=dtype)
    sc, sh = np.float32(scale), np.float32(shift)
    for a in range(0, n, _CHUNK):
        cnt = min(_CHUNK, n - a)
        z = standard_normals(key, a, cnt).astype(np.float32)
        out[a:a + cnt] = torch.from_numpy(z * sc + sh).to(dtype)
    return out.view(*spec.shape)


_lib = None


def _device_tensor(key: int, spec: TensorSpec, scale: float, shift: float, dtype: torch.dtype,
                   device: torch.device) -> torch.Tensor:
    global _lib
    from ..csrc import build
    if _lib is None:
        _lib = build.load_library("random_init")
        _lib.tl_random_fill.restype = ctypes.c_int
    kind = 2 if spec.integer else {torch.float32: 0, torch.bfloat16: 1}[dtype]
    out = torch.empty(spec.shape, dtype=torch.int32 if spec.integer else dtype, device=device)
    c = _consts()
    with torch.cuda.device(device):
        rc = _lib.tl_random_fill(ctypes.c_void_p(out.data_ptr()), ctypes.c_longlong(out.numel()),
                                 ctypes.c_ulonglong(key), ctypes.c_int(kind), ctypes.c_float(scale),
                                 ctypes.c_float(shift), ctypes.c_int(INT_MODULUS), ctypes.byref(c),
                                 ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    if rc != 0:
        raise RuntimeError(f"random weights: the fill kernel failed with code {rc}")
    return out


def random_tensor(name: str, spec: TensorSpec, seed: int, dtype: torch.dtype,
                  device: str | torch.device = "cpu") -> torch.Tensor:
    """One tensor.  Vectors (one dimension) are taken to be norm weights.  A value is drawn in
    double precision, rounded to 32-bit, scaled (and shifted) in 32-bit and then rounded to
    `dtype` (float32, bfloat16; float16 on the host only).  The same bits on a CUDA device and
    on the host."""
    dev = torch.device(device)
    key = tensor_key(seed, name)
    scale, shift = (NORM_STD, 1.0) if len(spec.shape) == 1 else (MATRIX_STD, 0.0)
    if dev.type == "cuda" and (spec.integer or dtype in (torch.float32, torch.bfloat16)):
        return _device_tensor(key, spec, scale, shift, dtype, dev)
    return _host_tensor(key, spec, scale, shift, dtype).to(dev)


def random_tensors(expected: Mapping[str, TensorSpec], seed: int, dtype: torch.dtype,
                   device: str | torch.device = "cpu") -> Iterator[Tuple[str, torch.Tensor]]:
    for name, spec in expected.items():
        yield name, random_tensor(name, spec, seed, dtype, device)


def write_random_model(config, out_dir: str, seed: int, dtype: torch.dtype = torch.bfloat16,
                       device: str | torch.device = "cpu") -> str:
    """Writes `config.json` and `model.safetensors` for `config` (a registered
    configuration object) into `out_dir` and returns the folder.  `device`: where the
    values are drawn (a CUDA device is much faster for large models; the file is the same)."""
    from ..engine.model import expected_tensors
    os.makedirs(out_dir, exist_ok=True)
    expected = expected_tensors(config.model_spec())
    d = config.to_dict()
    d["torch_dtype"] = {torch.bfloat16: "bfloat16", torch.float32: "float32",
                        torch.float16: "float16"}[dtype]
    with open(os.path.join(out_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(d, f, indent=1)
    write_safetensors(os.path.join(out_dir, "model.safetensors"),
                      [(n, t.cpu()) for n, t in random_tensors(expected, seed, dtype, device)],
                      metadata={"format": "pt", "seed": str(seed)})
    return out_dir
