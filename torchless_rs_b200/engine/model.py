"""A decoder built from a `ModelSpec`: embedding, layers made of registered parts,
final norm and head.  Nothing here knows an architecture's name
(reference for the Mistral arrangement: src/model/mod.rs:353-468)."""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..config.errors import ConfigError
from ..config.spec import LayerSpec, ModelSpec, PartSpec
from ..csrc import ops
from ..parts import lookup
from ..parts.linear import Matmul
from ..parts.runtime import Runtime
from ..weights.loader import TensorSpec


def _block_class(layer: LayerSpec) -> type:
    """The layer's block class, after checking that the layer gives exactly the norms
    that this kind of block takes."""
    cls = lookup("block", layer.block.kind)
    roles = tuple(getattr(cls, "norm_roles", ()))
    if set(roles) != set(layer.norms):
        raise ConfigError(
            f"layer '{layer.prefix}': a '{layer.block.kind}' block takes the norms "
            f"{sorted(roles)}, the layer gives {sorted(layer.norms)}")
    return cls


def expected_tensors(spec: ModelSpec) -> Dict[str, TensorSpec]:
    """Every tensor name the model asks for, with its shape.  Parts say what they
    need through their `expected_tensors(spec, prefix)` class method; the prefix of
    each part comes from the layer's `names`."""
    out: Dict[str, TensorSpec] = {
        spec.embedding_name: TensorSpec((spec.vocab_size, spec.hidden_size))}
    if spec.position_table_name is not None:
        out[spec.position_table_name] = TensorSpec((spec.max_positions, spec.hidden_size))
    for layer in spec.layers:
        _block_class(layer)
        for table, ps, role in (
                [("mixer", layer.mixer, "mixer"), ("feed_forward", layer.feed_forward, "feed_forward")] +
                [("norm", ps, role) for role, ps in layer.norms.items()]):
            out.update(lookup(table, ps.kind).expected_tensors(_own(ps, layer), layer.tensor_prefix(role)))
    out.update(lookup("norm", spec.final_norm.kind).expected_tensors(spec.final_norm,
                                                                     spec.final_norm_prefix))
    if not spec.tie_head_to_embedding:
        out[spec.head_name] = TensorSpec((spec.vocab_size, spec.hidden_size))
    return out


def _own(ps, layer: LayerSpec):
    """A mixer that reads another layer's cache keeps none of its own."""
    if layer.cache_from is not None and ps is layer.mixer:
        return PartSpec(ps.kind, {**ps.params, "own_cache": False})
    return ps


class DecoderModel:
    def __init__(self, spec: ModelSpec, rt: Runtime):
        spec.validate()
        self.spec = spec
        self.rt = rt
        self.matmul = Matmul(rt)
        self.blocks = []
        self.mixers = []
        for layer in spec.layers:
            block_cls = _block_class(layer)
            position = (lookup("position", layer.position.kind)(layer.position, rt)
                        if layer.position is not None else None)
            mixer = lookup("mixer", layer.mixer.kind)(
                _own(layer.mixer, layer), layer.tensor_prefix("mixer"), rt, position=position)
            ff = lookup("feed_forward", layer.feed_forward.kind)(
                layer.feed_forward, layer.tensor_prefix("feed_forward"), rt)
            norms = {role: lookup("norm", ps.kind)(ps, layer.tensor_prefix(role), rt)
                     for role, ps in layer.norms.items()}
            self.blocks.append(block_cls(layer.block, rt, mixer, ff, norms))
            self.mixers.append(mixer)
        self.final_norm = lookup("norm", spec.final_norm.kind)(
            spec.final_norm, spec.final_norm_prefix, rt)
        self.embedding: Optional[torch.Tensor] = None
        self.position_table: Optional[torch.Tensor] = None
        self.head: Optional[torch.Tensor] = None
        # a part whose forward reads host-side values of the batch cannot be replayed from a
        # recorded graph; it says so by not setting `graph_safe`
        self.graph_safe = all(getattr(p, "graph_safe", False)
                              for b in self.blocks for p in (b.mixer, b.feed_forward))

    @staticmethod
    def _parts_of(block) -> list:
        return [*block.norms.values(), block.mixer, block.feed_forward]

    # ---- weights ---------------------------------------------------------------------
    def tensors(self) -> Dict[str, TensorSpec]:
        return expected_tensors(self.spec)

    def load(self, weights: Dict[str, torch.Tensor]) -> None:
        self.embedding = self.rt.matrix(weights[self.spec.embedding_name])
        if self.spec.position_table_name is not None:
            self.position_table = self.rt.matrix(weights[self.spec.position_table_name])
        for b in self.blocks:
            for part in self._parts_of(b):
                part.load(weights)
        self.final_norm.load(weights)
        self.head = (self.embedding if self.spec.tie_head_to_embedding
                     else self.rt.matrix(weights[self.spec.head_name]))

    def weight_bytes(self) -> int:
        seen, total = set(), 0
        def add(t):
            nonlocal total
            if t is not None and t.data_ptr() not in seen:
                seen.add(t.data_ptr())
                total += t.numel() * t.element_size()
        add(self.embedding); add(self.head); add(self.position_table)
        for b in self.blocks:
            for part in self._parts_of(b):
                for v in vars(part).values():
                    if isinstance(v, torch.Tensor):
                        add(v)
        return total

    # ---- cache ------------------------------------------------------------------------
    # A cache belongs to a place in the order, not to a layer: a layer that is named twice
    # runs twice per token and keeps keys and values of both passes apart.
    def cache_requests(self) -> List[object]:
        """One request per entry of the order (None where the entry keeps no cache)."""
        return [self.mixers[i].cache_request() for i in self.spec.order]

    def bind_cache(self, cache) -> None:
        self.views = []
        last_run = {}     # layer -> the latest entry of the order that ran it
        for k, i in enumerate(self.spec.order):
            src = self.spec.layers[i].cache_from
            self.views.append(cache.view(k) if src is None else cache.view(last_run[src]))
            last_run[i] = k

    # ---- one step -----------------------------------------------------------------------
    def forward(self, batch) -> Optional[torch.Tensor]:
        """Runs the step's tokens through the layers in the spec's order and returns
        the logits [wanted, vocab] in 32-bit at `batch.want_rows` (None if none)."""
        rt, ws = self.rt, self.rt.workspace
        T, H = batch.n_tokens, self.spec.hidden_size
        x = ws.get("stream", (T, H), torch.float32)
        rt.ops.embed(batch.tokens, self.embedding, x, batch.token_from, batch.token_src,
                     scale=self.spec.embedding_scale, position_table=self.position_table,
                     token_pos=batch.token_pos)
        order = self.spec.order
        carry = None
        for k, i in enumerate(order):
            self.mixers[i].bind_cache(self.views[k])
            block = self.blocks[i]
            if not getattr(block, "takes_carry", False):
                block.forward(x, batch)       # the plain interface of a block
                carry = None
                continue
            # A block that `takes_carry` may get its first norm's input prepared by the block
            # before it, and prepare the next block's: `first_norm` names the norm in question.
            nxt = self.blocks[order[k + 1]] if k + 1 < len(order) else None
            next_norm = getattr(nxt, "first_norm", None) if getattr(nxt, "takes_carry", False) else None
            carry = block.forward(x, batch, carry, next_norm)
        if batch.n_want == 0:
            return None
        xn = ws.get("head_normed", (batch.n_want, H), rt.act_dtype)
        self.final_norm(x, xn, rows=batch.want_rows)
        logits = ws.get("logits", (batch.n_want, self.spec.vocab_size), torch.float32)
        self.matmul(xn, self.head, logits, ops.MODE_STORE_F32)
        if self.spec.logit_softcap is not None:
            rt.ops.softcap(logits, self.spec.logit_softcap)
        return logits
