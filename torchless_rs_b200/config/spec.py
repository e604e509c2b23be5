"""The description of a model as data: which parts each layer is made of, with
their sizes and constants, and the order in which layers run.

A configuration class turns its config.json keys into a `ModelSpec`; the engine
builds parts from it through the part registries and never asks which
architecture it is running.  The reference fixes one arrangement per model file
(src/model/modules/layer.rs:28-56 for Mistral); here the arrangement is a value.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping, Optional, Sequence


@dataclass(frozen=True)
class PartSpec:
    """One part: the name it is registered under and its own parameters."""
    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)

    def get(self, key: str, default: Any = None) -> Any:
        return self.params.get(key, default)


@dataclass(frozen=True)
class LayerSpec:
    """One layer.  `prefix` is the tensor-name prefix of its weights.  `cache_from`
    names another layer (index into `ModelSpec.layers`) whose cache this layer's
    mixer reads instead of keeping one of its own."""
    prefix: str
    block: PartSpec
    mixer: PartSpec
    feed_forward: PartSpec
    mixer_norm: PartSpec
    feed_forward_norm: PartSpec
    position: Optional[PartSpec] = None
    cache_from: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    """A whole decoder.  `order` lists indices into `layers` in the order in which
    they run; an index may appear more than once."""
    hidden_size: int
    vocab_size: int
    embedding_name: str
    head_name: str
    tie_head_to_embedding: bool
    final_norm: PartSpec
    final_norm_prefix: str
    layers: Sequence[LayerSpec]
    order: Sequence[int]
    stop_token_ids: Sequence[int] = ()

    def validate(self) -> None:
        from .errors import ConfigError
        n = len(self.layers)
        if n == 0:
            raise ConfigError("a model needs at least one layer")
        for i in self.order:
            if not 0 <= i < n:
                raise ConfigError(f"layer order names layer {i}, but there are {n} layers")
        first_run = {}
        for step, i in enumerate(self.order):
            first_run.setdefault(i, step)
        for i, layer in enumerate(self.layers):
            src = layer.cache_from
            if src is None:
                continue
            if not 0 <= src < n or src == i:
                raise ConfigError(f"layer {i} reads the cache of layer {src}, which does not exist")
            if self.layers[src].cache_from is not None:
                raise ConfigError(f"layer {i} reads the cache of layer {src}, which keeps none itself")
            if i in first_run and (src not in first_run or first_run[src] > first_run[i]):
                raise ConfigError(f"layer {i} reads the cache of layer {src} before that layer has run")
