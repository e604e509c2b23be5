"""What every part is given when it is built: the device, the activation type,
the kernels of that type, and a workspace of reusable buffers."""
from __future__ import annotations

from typing import Dict, Tuple

import torch

from ..csrc import ops


class Workspace:
    """Named scratch buffers that are kept between steps.  A buffer grows when a
    step asks for more than it holds and is never shrunk, so once the largest step
    has run, addresses stay the same (which CUDA graphs rely on)."""

    def __init__(self, device: torch.device):
        self.device = device
        self._bufs: Dict[Tuple[str, torch.dtype], torch.Tensor] = {}
        self.generation = 0   # goes up whenever a buffer moves; recorded CUDA graphs are then stale
        self._views: Dict[tuple, torch.Tensor] = {}

    def get(self, name: str, shape, dtype: torch.dtype) -> torch.Tensor:
        # the view of a buffer for a shape is kept: making one costs 4 us, and a layer asks for nine
        vkey = (name, dtype, tuple(shape))
        view = self._views.get(vkey)
        if view is not None:
            return view
        n = 1
        for s in shape:
            n *= int(s)
        key = (name, dtype)
        buf = self._bufs.get(key)
        if buf is None or buf.numel() < n:
            buf = torch.empty(max(n, 1), dtype=dtype, device=self.device)
            self._bufs[key] = buf
            self.generation += 1
            for k in [k for k in self._views if k[0] == name and k[1] == dtype]:
                del self._views[k]          # they show the buffer that was replaced
        if len(self._views) > 4096:
            self._views.clear()
        view = buf[:n].view(*shape)
        self._views[vkey] = view
        return view

    def bytes_held(self) -> int:
        return sum(b.numel() * b.element_size() for b in self._bufs.values())


class Runtime:
    def __init__(self, device="cuda:0", act_dtype: torch.dtype = torch.bfloat16):
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise ops.KernelError(
                f"device '{device}': this package runs on CUDA devices only; there is no CPU path")
        if not torch.cuda.is_available():
            raise ops.KernelError("no CUDA device is available; there is no CPU path")
        if act_dtype not in (torch.float32, torch.bfloat16):
            raise ValueError(f"dtype must be float32 or bfloat16, got {act_dtype}")
        self.act_dtype = act_dtype
        self.ops = ops.core_ops(act_dtype)
        self.workspace = Workspace(self.device)

    @property
    def is_f32(self) -> bool:
        return self.act_dtype == torch.float32

    def matrix(self, t: torch.Tensor) -> torch.Tensor:
        """A weight matrix or table as the matrix kernels read it: on the device, in
        the activation type."""
        return self.stack([t])

    def stack(self, tensors) -> torch.Tensor:
        """Several stored matrices of one width, one below the other, as one matrix on the device in
        the activation type (q, k and v; gate and up).  Each is copied to the device as stored and
        converted at its place by a kernel; no joined copy is made."""
        width = tensors[0].shape[1:]
        for t in tensors:
            if t.shape[1:] != width:
                raise ValueError("stacked matrices must have one width")
        rows = sum(int(t.shape[0]) for t in tensors)
        out = torch.empty((rows, *width), dtype=self.act_dtype, device=self.device)
        at = 0
        for t in tensors:
            n = int(t.shape[0])
            raw = t.contiguous().to(self.device)          # as stored
            if raw.dtype == self.act_dtype:
                out[at:at + n].copy_(raw)
            else:
                self.ops.convert_into(raw, out[at:at + n])
            at += n
        return out

    def vector(self, t: torch.Tensor) -> torch.Tensor:
        """A norm weight: 32-bit if it was stored so or if the whole model runs in
        32-bit, else bfloat16 as stored."""
        dt = torch.float32 if (self.is_f32 or t.dtype == torch.float32) else torch.bfloat16
        return t.to(device=self.device, dtype=dt).contiguous()
