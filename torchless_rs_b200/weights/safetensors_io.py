"""Reading and writing of the safetensors container.

Layout, as the reference reads it (src/loader/formats/safetensors.rs:196-280):
an unsigned 64-bit little-endian header size, a JSON object from tensor name to
{dtype, shape, data_offsets} (plus an optional "__metadata__"), then the raw
tensor bytes; offsets count from the end of the header.  The checks are those
of the reference (file too small :204, header size :215-221, JSON :225-230,
unknown dtype :253-255, data beyond the file :345-353) plus overlapping and
duplicate entries.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, Iterable, List, Tuple

import torch

from .errors import SafetensorsFormatError

_DTYPES = {
    "F64": (torch.float64, 8), "F32": (torch.float32, 4), "F16": (torch.float16, 2),
    "BF16": (torch.bfloat16, 2), "I64": (torch.int64, 8), "I32": (torch.int32, 4),
    "I16": (torch.int16, 2), "I8": (torch.int8, 1), "U8": (torch.uint8, 1),
    "BOOL": (torch.bool, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}


class SafetensorsFile:
    """One memory-mapped file.  `tensor(name)` gives a CPU tensor that views the
    mapping (no copy); keep the file object alive while such tensors are used."""

    def __init__(self, path: str):
        self.path = path
        size = os.path.getsize(path)
        if size < 8:
            raise SafetensorsFormatError(f"{path}: file too small for a safetensors header")
        self._fh = open(path, "rb")
        self._map = mmap.mmap(self._fh.fileno(), 0, access=mmap.ACCESS_READ)
        (hlen,) = struct.unpack("<Q", self._map[:8])
        if hlen == 0 or 8 + hlen > size:
            raise SafetensorsFormatError(f"{path}: header size {hlen} does not fit the file ({size} bytes)")
        try:
            header = json.loads(self._map[8:8 + hlen].decode("utf-8"),
                                object_pairs_hook=self._no_duplicates)
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsFormatError(f"{path}: header is not valid JSON ({e})") from e
        if not isinstance(header, dict):
            raise SafetensorsFormatError(f"{path}: header must be a JSON object")
        self.metadata = header.pop("__metadata__", {}) or {}
        self._data_start = 8 + hlen
        data_len = size - self._data_start
        self.entries: Dict[str, Tuple[torch.dtype, Tuple[int, ...], int, int]] = {}
        spans: List[Tuple[int, int, str]] = []
        for name, info in header.items():
            try:
                dt, shape, (lo, hi) = info["dtype"], tuple(int(s) for s in info["shape"]), info["data_offsets"]
            except (KeyError, TypeError, ValueError) as e:
                raise SafetensorsFormatError(f"{path}: entry '{name}' is malformed ({e})") from e
            if dt not in _DTYPES:
                raise SafetensorsFormatError(f"{path}: entry '{name}' has unknown dtype '{dt}'")
            tdt, isz = _DTYPES[dt]
            count = 1
            for s in shape:
                count *= s
            if lo < 0 or hi < lo or hi > data_len:
                raise SafetensorsFormatError(
                    f"{path}: entry '{name}' spans bytes {lo}..{hi}, beyond the {data_len} bytes of data")
            if hi - lo != count * isz:
                raise SafetensorsFormatError(
                    f"{path}: entry '{name}' holds {hi - lo} bytes, its shape {list(shape)} needs {count * isz}")
            self.entries[name] = (tdt, shape, lo, hi)
            spans.append((lo, hi, name))
        spans.sort()
        for (l0, h0, n0), (l1, h1, n1) in zip(spans, spans[1:]):
            if l1 < h0 and h1 > l1:
                raise SafetensorsFormatError(f"{path}: entries '{n0}' and '{n1}' overlap")

    @staticmethod
    def _no_duplicates(pairs):
        out = {}
        for k, v in pairs:
            if k in out:
                raise SafetensorsFormatError(f"tensor '{k}' appears twice in the header")
            out[k] = v
        return out

    def names(self) -> List[str]:
        return list(self.entries)

    def shape(self, name: str) -> Tuple[int, ...]:
        return self.entries[name][1]

    def dtype(self, name: str) -> torch.dtype:
        return self.entries[name][0]

    def tensor(self, name: str) -> torch.Tensor:
        tdt, shape, lo, hi = self.entries[name]
        if hi == lo:
            return torch.empty(shape, dtype=tdt)
        buf = memoryview(self._map)[self._data_start + lo:self._data_start + hi]
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")  # the mapping is read-only; nothing writes through it
            t = torch.frombuffer(buf, dtype=tdt)
        return t.reshape(shape)

    def close(self) -> None:
        try:
            self._map.close()
        except BufferError:
            pass  # tensors still view the mapping; it is released with them
        self._fh.close()


def write_safetensors(path: str, tensors: Iterable[Tuple[str, torch.Tensor]],
                      metadata: Dict[str, str] | None = None) -> None:
    """Writes name/tensor pairs in the given order; each tensor starts on an
    8-byte boundary relative to the data section.  `tensors` may be a generator
    of a size that does not fit memory at once: shapes are taken in a first pass
    only if it is a list, so pass a list of (name, tensor) or a callable-backed
    sequence."""
    items = list(tensors)
    header: Dict[str, dict] = {}
    if metadata:
        header["__metadata__"] = dict(metadata)
    off = 0
    for name, t in items:
        if name in header:
            raise SafetensorsFormatError(f"tensor '{name}' given twice")
        if t.dtype not in _NAMES:
            raise SafetensorsFormatError(f"tensor '{name}' has dtype {t.dtype}, which safetensors cannot hold")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape),
                        "data_offsets": [off, off + nbytes]}
        off += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for _, t in items:
            c = t.detach().contiguous().cpu()
            if c.numel():
                f.write(c.view(torch.uint8).numpy().tobytes() if c.dim() else
                        c.reshape(1).view(torch.uint8).numpy().tobytes())
    os.replace(tmp, path)
