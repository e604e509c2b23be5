"""The Python entry point: load a model folder, generate, or drive steps by hand.

    import torchless_rs_b200 as tl
    m = tl.load("model_dir", dtype="bfloat16", max_tokens=8192)
    out = m.generate([[1, 5, 9], [1, 7]], max_tokens=16, temperature=0.0)

(The reference's library surface, for comparison: docs/library.md:21-139,
src/lib.rs:54-91: load parameters, build the model, create a state, call forward
and a sampler.)"""
from __future__ import annotations

from typing import Callable, List, Optional, Sequence, Union

import torch

from .config import load_config
from .engine.engine import Engine
from .engine.generate import GenerationResult, generate as _generate
from .engine.model import expected_tensors
from .parts.runtime import Runtime
from .sampling.params import SamplingParams
from .weights.loader import load_checked
from .weights.random_init import random_tensors

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32,
           "fp32": torch.float32, "f32": torch.float32}


def parse_dtype(dtype: Union[str, torch.dtype]) -> torch.dtype:
    if isinstance(dtype, torch.dtype):
        if dtype in (torch.bfloat16, torch.float32):
            return dtype
    elif str(dtype).lower() in _DTYPES:
        return _DTYPES[str(dtype).lower()]
    raise ValueError(f"dtype must be bfloat16 or float32, got {dtype!r}")


class OverlappedReader:
    """Copies selected tokens to pinned host memory without waiting; `finish` waits for
    that copy only.  Two buffers in rotation, since one step is launched ahead."""
    overlapped = True

    def __init__(self, rows: int = 256):
        self.bufs = [torch.empty(rows, dtype=torch.int32, pin_memory=True) for _ in range(3)]
        self.events = [torch.cuda.Event() for _ in range(3)]
        self.turn = 0
        self.bytes_copied = 0   # device-to-host bytes so far

    def start(self, selected: torch.Tensor):
        n = selected.numel()
        self.turn = (self.turn + 1) % 3
        if self.bufs[self.turn].numel() < n:
            self.bufs = [torch.empty(2 * n, dtype=torch.int32, pin_memory=True) for _ in range(3)]
        buf, ev = self.bufs[self.turn], self.events[self.turn]
        buf[:n].copy_(selected, non_blocking=True)
        self.bytes_copied += 4 * n
        ev.record()
        return buf, n, ev

    def finish(self, handle) -> List[int]:
        buf, n, ev = handle
        ev.synchronize()
        return buf[:n].tolist()


class Model:
    """A loaded model with its cache.  `config` is the typed configuration;
    `engine` gives `step`, `start_sequences`, `end_sequences`."""

    def __init__(self, config, engine: Engine):
        self.config = config
        self.engine = engine
        self._sampler = None
        self._reader = None

    @property
    def sampler(self):
        """Built at first use, so that replaying logits never compiles the sampling kernels."""
        if self._sampler is None:
            from .sampling.sampler import Sampler
            self._sampler = Sampler(self.engine.rt.device)
        return self._sampler

    def generate(self, prompts: Sequence[Sequence[int]], max_tokens: int = 16,
                 temperature: float = 0.0, top_k: Optional[int] = None,
                 top_p: Optional[float] = None, stop_ids: Optional[Sequence[int]] = None,
                 seed: int = 0, on_token: Optional[Callable[[int, int], None]] = None,
                 max_batch: Optional[int] = None) -> List[GenerationResult]:
        """Token ids in (host lists), token ids out.  `stop_ids` defaults to the
        configuration's end tokens; pass () for none."""
        params = SamplingParams(temperature=temperature, top_k=top_k, top_p=top_p)
        if stop_ids is None:
            stop_ids = self.engine.spec.stop_token_ids
        if self._reader is None:
            self._reader = OverlappedReader()
        results = _generate(self.engine, self.sampler.select, prompts, max_tokens, params, stop_ids,
                            seed, on_token, max_batch=max_batch, reader=self._reader)
        self.engine.check_kernels()
        return results

    def step(self, slots, tokens, want="last"):
        return self.engine.step(slots, tokens, want)

    def prefill(self, slots, prompts, tokens_per_step=None):
        """The logits at each prompt's last token; many tokens go in several steps."""
        return self.engine.prefill(slots, prompts, tokens_per_step)

    def start_sequences(self, count: int):
        return self.engine.start_sequences(count)

    def end_sequences(self, slots) -> None:
        self.engine.end_sequences(slots)

    def truncate(self, slot: int, length: int) -> None:
        """Rolls the sequence of `slot` back to its first `length` tokens."""
        self.engine.truncate(slot, length)

    def reset(self, slot: int) -> None:
        """Rolls the sequence of `slot` back to empty; the slot stays held."""
        self.engine.reset(slot)


def _default_max_tokens(config) -> int:
    return int(getattr(config, "max_position_embeddings", 4096))


def load(model_dir: str, dtype: Union[str, torch.dtype] = "bfloat16",
         max_tokens: Optional[int] = None, max_batch: Optional[int] = None,
         max_seq_len: Optional[int] = None, device: str = "cuda:0",
         random_weights: bool = False, seed: int = 0) -> Model:
    """Loads `config.json` and the safetensors weights of `model_dir`.  The model
    class is chosen by config.json through the architecture registry.  With
    `random_weights` the folder needs config.json only: the weights are drawn from `seed`
    (the same values that `write_random_model` writes for that seed)."""
    config = load_config(model_dir)
    if random_weights:
        return from_random(config, seed, dtype, max_tokens, max_batch, max_seq_len, device)
    spec = config.model_spec()
    rt = Runtime(device, parse_dtype(dtype))
    weights, source = load_checked(model_dir, expected_tensors(spec), rt.act_dtype)
    try:
        engine = Engine(spec, weights, rt, max_tokens or _default_max_tokens(config),
                        max_batch, max_seq_len)
    finally:
        del weights
        source.close()
    return Model(config, engine)


def from_random(config, seed: int = 0, dtype: Union[str, torch.dtype] = "bfloat16",
                max_tokens: Optional[int] = None, max_batch: Optional[int] = None,
                max_seq_len: Optional[int] = None, device: str = "cuda:0") -> Model:
    """A model with random weights drawn on the device, without a model folder
    (for measurements at sizes whose folder would be tens of gigabytes)."""
    spec = config.model_spec()
    adt = parse_dtype(dtype)
    rt = Runtime(device, adt)

    exp = expected_tensors(spec)
    weights = {n: t for n, t in random_tensors(exp, seed, adt, rt.device)}
    engine = Engine(spec, weights, rt, max_tokens or _default_max_tokens(config), max_batch,
                    max_seq_len)
    del weights
    torch.cuda.empty_cache()
    return Model(config, engine)
