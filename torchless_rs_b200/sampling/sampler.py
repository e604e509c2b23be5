"""Token selection on the device (kernels in csrc/sampling.cu).

The reference selects on the host, one sequence at a time: arg-max, or temperature, top-k,
softmax, top-p and an inverse-CDF draw in that order (src/sampler/mod.rs:17-238).  Here every row
of a batch has its own parameters and its own uniform number."""
from __future__ import annotations

from typing import Optional, Sequence

import torch

from ..csrc import ops
from .params import SamplingParams


class Sampler:
    def __init__(self, device: torch.device, max_rows: int = 256):
        self.device = torch.device(device)
        self.ops = ops.sampling_ops()
        self._resize(max_rows)

    def _resize(self, rows: int) -> None:
        self.max_rows = rows
        self.out = torch.empty(rows, dtype=torch.int32, device=self.device)
        # pinned staging in rotation: a select may be enqueued before the previous copy has run
        self.uniform_hosts = [torch.empty(rows, dtype=torch.float32, pin_memory=True) for _ in range(4)]
        self.uniform_events = [None] * 4
        self.turn = 0
        self.uniform_dev = torch.empty(rows, dtype=torch.float32, device=self.device)

    def select(self, logits: torch.Tensor, params: SamplingParams,
               uniforms: Optional[Sequence[float]] = None) -> torch.Tensor:
        """One token per row of `logits` [rows, vocab] (32-bit, on the device);
        returns int32 [rows] on the device.  `uniforms`: one number in [0, 1) per row,
        needed unless greedy."""
        rows = logits.shape[0]
        if rows > self.max_rows:
            self._resize(max(rows, 2 * self.max_rows))
        out = self.out[:rows]
        if params.is_greedy:
            self.ops.argmax(logits, out)
            return out
        if uniforms is None or len(uniforms) != rows:
            raise ValueError("sampling with a temperature needs one uniform number per row")
        self.turn = (self.turn + 1) % 4
        if self.uniform_events[self.turn] is not None:
            self.uniform_events[self.turn].synchronize()
        host = self.uniform_hosts[self.turn]
        host[:rows] = torch.as_tensor(list(uniforms), dtype=torch.float32)
        self.uniform_dev[:rows].copy_(host[:rows], non_blocking=True)
        ev = self.uniform_events[self.turn] or torch.cuda.Event()
        ev.record()
        self.uniform_events[self.turn] = ev
        self.ops.sample(logits, float(params.temperature), int(params.top_k or 0),
                        float(params.top_p if params.top_p is not None else 0.0),
                        self.uniform_dev, out)
        return out
