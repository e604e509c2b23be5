"""A decoder built from a `ModelSpec`: embedding, layers made of registered parts,
final norm and head.  Nothing here knows an architecture's name
(reference for the Mistral arrangement: src/model/mod.rs:353-468)."""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..config.spec import LayerSpec, ModelSpec
from ..csrc import ops
from ..parts import lookup
from ..parts.linear import Matmul
from ..parts.runtime import Runtime
from ..weights.loader import TensorSpec


def expected_tensors(spec: ModelSpec) -> Dict[str, TensorSpec]:
    """Every tensor name the model asks for, with its shape.  Parts say what they
    need through their `expected_tensors(spec, prefix)` class method."""
    out: Dict[str, TensorSpec] = {
        spec.embedding_name: TensorSpec((spec.vocab_size, spec.hidden_size))}
    for layer in spec.layers:
        for table, ps, prefix in (
                ("norm", layer.mixer_norm, f"{layer.prefix}.input_layernorm"),
                ("mixer", layer.mixer, f"{layer.prefix}.self_attn"),
                ("norm", layer.feed_forward_norm, f"{layer.prefix}.post_attention_layernorm"),
                ("feed_forward", layer.feed_forward, f"{layer.prefix}.mlp")):
            out.update(lookup(table, ps.kind).expected_tensors(_own(ps, layer), prefix))
    out.update(lookup("norm", spec.final_norm.kind).expected_tensors(spec.final_norm,
                                                                     spec.final_norm_prefix))
    if not spec.tie_head_to_embedding:
        out[spec.head_name] = TensorSpec((spec.vocab_size, spec.hidden_size))
    return out


def _own(ps, layer: LayerSpec):
    """A mixer that reads another layer's cache keeps none of its own."""
    if layer.cache_from is not None and ps is layer.mixer:
        from ..config.spec import PartSpec
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
            position = (lookup("position", layer.position.kind)(layer.position, rt)
                        if layer.position is not None else None)
            mixer = lookup("mixer", layer.mixer.kind)(
                _own(layer.mixer, layer), f"{layer.prefix}.self_attn", rt, position=position)
            ff = lookup("feed_forward", layer.feed_forward.kind)(
                layer.feed_forward, f"{layer.prefix}.mlp", rt)
            n1 = lookup("norm", layer.mixer_norm.kind)(
                layer.mixer_norm, f"{layer.prefix}.input_layernorm", rt)
            n2 = lookup("norm", layer.feed_forward_norm.kind)(
                layer.feed_forward_norm, f"{layer.prefix}.post_attention_layernorm", rt)
            self.blocks.append(lookup("block", layer.block.kind)(layer.block, rt, mixer, ff, n1, n2))
            self.mixers.append(mixer)
        self.final_norm = lookup("norm", spec.final_norm.kind)(
            spec.final_norm, spec.final_norm_prefix, rt)
        self.embedding: Optional[torch.Tensor] = None
        self.head: Optional[torch.Tensor] = None
        # a part whose forward reads host-side values of the batch cannot be replayed from a
        # recorded graph; it says so by not setting `graph_safe`
        self.graph_safe = all(getattr(p, "graph_safe", False)
                              for b in self.blocks for p in (b.mixer, b.feed_forward))

    # ---- weights ---------------------------------------------------------------------
    def tensors(self) -> Dict[str, TensorSpec]:
        return expected_tensors(self.spec)

    def load(self, weights: Dict[str, torch.Tensor]) -> None:
        self.embedding = self.rt.matrix(weights[self.spec.embedding_name])
        for b in self.blocks:
            for part in (b.mixer_norm, b.mixer, b.feed_forward_norm, b.feed_forward):
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
        add(self.embedding); add(self.head)
        for b in self.blocks:
            for part in (b.mixer_norm, b.mixer, b.feed_forward_norm, b.feed_forward):
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
        rt.ops.embed(batch.tokens, self.embedding, x, batch.token_from, batch.token_src)
        order = self.spec.order
        carry = None
        for k, i in enumerate(order):
            self.mixers[i].bind_cache(self.views[k])
            nxt = self.blocks[order[k + 1]] if k + 1 < len(order) else None
            # the next block takes a prepared norm input only if its mixer can use one
            next_norm = (nxt.mixer_norm if nxt is not None
                         and getattr(nxt.mixer, "accepts_carry", False) else None)
            carry = self.blocks[i].forward(x, batch, carry, next_norm)
        if batch.n_want == 0:
            return None
        xn = ws.get("head_normed", (batch.n_want, H), rt.act_dtype)
        self.final_norm(x, xn, rows=batch.want_rows)
        logits = ws.get("logits", (batch.n_want, self.spec.vocab_size), torch.float32)
        self.matmul(xn, self.head, logits, ops.MODE_STORE_F32)
        return logits
