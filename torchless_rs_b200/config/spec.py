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
    """One layer.

    `norms` maps a role to a norm; which roles exist is the block kind's business (a
    block class lists them as `norm_roles`; the pre-norm block takes "mixer_norm" and
    "feed_forward_norm").  `names` gives, for "mixer", "feed_forward" and every norm
    role, the name under `prefix` that its tensors carry: the weights of role r are
    called `<prefix>.<names[r]>.*`, so an architecture with other tensor names is a
    matter of data.  `cache_from` names another layer (index into `ModelSpec.layers`)
    whose cache this layer's mixer reads instead of keeping one of its own."""
    prefix: str
    block: PartSpec
    mixer: PartSpec
    feed_forward: PartSpec
    norms: Mapping[str, PartSpec]
    names: Mapping[str, str]
    position: Optional[PartSpec] = None
    cache_from: Optional[int] = None

    def tensor_prefix(self, role: str) -> str:
        from .errors import ConfigError
        if role not in self.names:
            raise ConfigError(f"layer '{self.prefix}': no tensor name is given for its '{role}'")
        name = self.names[role]
        return f"{self.prefix}.{name}" if name else self.prefix


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
    # What happens to the stream between the embedding table and the first layer, and to the
    # logits after the head.  Every architecture sets what it has; the defaults do nothing.
    embedding_scale: float = 1.0                 # the embedded rows are multiplied by this
    position_table_name: Optional[str] = None    # a learned table [max_positions, hidden] whose row
    max_positions: int = 0                       #   at each token's position is added to the stream
    logit_softcap: Optional[float] = None        # logits <- cap * tanh(logits / cap)

    def validate(self) -> None:
        from .errors import ConfigError
        n = len(self.layers)
        if n == 0:
            raise ConfigError("a model needs at least one layer")
        if self.position_table_name is not None and self.max_positions <= 0:
            raise ConfigError("a position table needs max_positions > 0")
        if self.logit_softcap is not None and not self.logit_softcap > 0:
            raise ConfigError("logit_softcap must be positive")
        for i, layer in enumerate(self.layers):
            for role in ("mixer", "feed_forward", *layer.norms):
                if role not in layer.names:
                    raise ConfigError(f"layer {i}: no tensor name is given for its '{role}'")
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
            # the owner's window decides which pages are still held: a reader may not look further back
            own_w, src_w = layer.mixer.get("window"), self.layers[src].mixer.get("window")
            if src_w and (not own_w or own_w > src_w):
                raise ConfigError(
                    f"layer {i} (window {own_w}) reads the cache of layer {src}, which only keeps a "
                    f"window of {src_w} keys")
