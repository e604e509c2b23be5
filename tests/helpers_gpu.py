"""Helpers of the GPU tests: load a tiny model into the engine, run requests cut in
different ways, compare with the plain implementation."""
from __future__ import annotations

import numpy as np
import torch

from plain import mistral_plain as plain
from tiny import CONFIGS, make_model_dir, read_weights_numpy, remove_model_dir

# Stated tolerances.  32-bit: the engine and the plain implementation differ only in
# the order of 32-bit sums.  bfloat16: activations between kernels and the cache are
# rounded to 8 bits of mantissa (relative 2^-9 each) while the plain implementation
# keeps 32-bit; a handful of roundings per layer on logits of size ~0.1-1.
TOL = {"float32": dict(atol=5e-5, rtol=1e-4), "bfloat16": dict(atol=0.0, rtol=0.0, rel_max=2.5e-2)}


def assert_close(got: np.ndarray, ref: np.ndarray, dtype: str, what: str = "") -> None:
    assert got.shape == ref.shape, f"{what}: shape {got.shape} vs {ref.shape}"
    assert np.isfinite(got).all(), f"{what}: non-finite logits"
    err = np.abs(got - ref)
    if dtype == "float32":
        bound = TOL[dtype]["atol"] + TOL[dtype]["rtol"] * np.abs(ref)
        bad = err > bound
        assert not bad.any(), (f"{what}: max err {err.max():.3e} at {np.unravel_index(err.argmax(), err.shape)}"
                               f" (first bad row {np.argwhere(bad)[0]})")
    else:
        scale = np.abs(ref).max()
        rows = err.max(axis=-1) / scale
        assert rows.max() <= TOL[dtype]["rel_max"], (
            f"{what}: max err / max|ref| = {rows.max():.3e} at row {rows.argmax()}")


class TinyModel:
    def __init__(self, cfg_name: str, dtype: str, seed: int = 0, max_tokens: int = 1024,
                 max_batch=None, store=None, cfg=None):
        """`store`: the type the folder's tensors are written in; by default 32-bit for a
        model that runs in 32-bit (so that products see full mantissas) and bfloat16 else."""
        import torchless_rs_b200 as tl
        self.cfg = dict(cfg if cfg is not None else CONFIGS[cfg_name])
        self.dtype = dtype
        if store is None:
            store = torch.float32 if dtype == "float32" else torch.bfloat16
        d = make_model_dir(self.cfg, seed, store)
        try:
            self.weights = read_weights_numpy(d)
            self.model = tl.load(d, dtype=dtype, max_tokens=max_tokens, max_batch=max_batch)
        finally:
            remove_model_dir(d)      # the folder is needed for loading only (real sizes take a gigabyte)
        self.engine = self.model.engine
        self._ref = {}

    def reference(self, tokens) -> np.ndarray:
        key = tuple(tokens)
        if key not in self._ref:
            self._ref[key] = plain.forward_logits(self.cfg, self.weights, list(tokens))
        return self._ref[key]

    def step_np(self, slots, tokens, want) -> np.ndarray:
        out = self.engine.step(slots, tokens, want)
        return out.float().cpu().numpy().copy()
