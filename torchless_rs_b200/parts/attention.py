"""Grouped-query attention over the paged cache, with an optional window
(reference: src/model/modules/attention.rs:46-135; the window's inequality is that
of src/model/models/gpt_oss.rs:168-176, which the reference's Mistral never applies).

One product gives q, k and v (their matrices are stacked at load time); one kernel
rotates q and k at each token's position and writes k and v into the cache pages;
attention then reads keys and values from the pages only, for prefill and decode
alike, so a position's result does not depend on the step that computes it."""
from __future__ import annotations

import math
from typing import Dict, Optional

import torch

from ..cache.requests import PagedKVRequest
from ..config.spec import PartSpec
from ..csrc import ops
from ..weights.loader import TensorSpec
from .linear import Matmul
from .registry import register_mixer
from .runtime import Runtime


@register_mixer("attention")
class Attention:
    """Parameters: `hidden_size`, `num_heads`, `num_kv_heads`, `head_dim`, `window`
    (None = all keys), `own_cache` (False for a layer that reads another layer's keys
    and values; it then has no k and v matrices).

    Interface of every mixer: `expected_tensors(spec, prefix)` (a class method), `load(weights)`, `cache_request()` (what
    it asks of the cache, or None), `bind_cache(view)` (the view of its own layer or
    of the layer it reads), and `forward(xn, residual, batch)`, which adds its
    output to the 32-bit `residual` in place."""
    graph_safe = True   # forward launches kernels whose arguments do not depend on host values


    def __init__(self, spec: PartSpec, prefix: str, rt: Runtime, position=None):
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.nh = int(p["num_heads"])
        self.nkv = int(p["num_kv_heads"])
        self.hd = int(p["head_dim"])
        self.window = int(p["window"]) if p.get("window") else None
        self.own_cache = bool(p.get("own_cache", True))
        if self.nh % self.nkv:
            raise ValueError(f"{self.nh} heads cannot share {self.nkv} key/value heads")
        if self.hd % 16 or not 16 <= self.hd <= 256:
            raise ValueError(f"head_dim {self.hd} is not supported (16 to 256 in steps of 16)")
        self.scale = 1.0 / math.sqrt(self.hd)
        self.prefix = prefix
        self.rt = rt
        self.position = position
        self.matmul = Matmul(rt)
        self.w_qkv: Optional[torch.Tensor] = None
        self.w_o: Optional[torch.Tensor] = None
        self.cache = None
        self.fast = None
        if not rt.is_f32:
            from ..csrc import attention_bf16
            self.fast = attention_bf16.AttentionBf16.get(self.hd)

    @property
    def qkv_cols(self) -> int:
        return (self.nh + (2 * self.nkv if self.own_cache else 0)) * self.hd

    @classmethod
    def expected_tensors(cls, spec: PartSpec, prefix: str) -> Dict[str, TensorSpec]:
        p = spec.params
        hidden, nh, nkv, hd = (int(p[k]) for k in ("hidden_size", "num_heads", "num_kv_heads", "head_dim"))
        t = {f"{prefix}.q_proj.weight": TensorSpec((nh * hd, hidden)),
             f"{prefix}.o_proj.weight": TensorSpec((hidden, nh * hd))}
        if p.get("own_cache", True):
            t[f"{prefix}.k_proj.weight"] = TensorSpec((nkv * hd, hidden))
            t[f"{prefix}.v_proj.weight"] = TensorSpec((nkv * hd, hidden))
        return t

    def load(self, weights: Dict[str, torch.Tensor]) -> None:
        p = self.prefix
        names = ["q_proj"] + (["k_proj", "v_proj"] if self.own_cache else [])
        self.w_qkv = self.rt.stack([weights[f"{p}.{n}.weight"] for n in names])
        self.w_o = self.rt.matrix(weights[f"{p}.o_proj.weight"])

    def cache_request(self):
        return PagedKVRequest(self.nkv, self.hd, self.window) if self.own_cache else None

    def bind_cache(self, view) -> None:
        self.cache = view

    accepts_carry = True   # `xn` may be a NormCarry; `emit` may ask for the next norm's input

    def forward(self, xn, residual: torch.Tensor, batch, emit=None) -> None:
        rt, ws = self.rt, self.rt.workspace
        T = residual.shape[0]
        c = self.cache
        qkv = ws.get("attn_qkv", (T, self.qkv_cols), torch.float32)
        q = ws.get("attn_q", (T, self.nh * self.hd), rt.act_dtype)
        pos = self.position
        rope = None
        if self.fast is not None and self.own_cache:
            # the product may rotate and write q, k and v itself (it does when K is split)
            from ..csrc.gemm_bf16 import RopeArgs
            rope = RopeArgs(q.data_ptr(), c.k_pages.data_ptr(), c.v_pages.data_ptr(),
                            batch.token_pos.data_ptr(), batch.token_seq.data_ptr(),
                            batch.seq_slot.data_ptr(), c.page_table.data_ptr(),
                            pos.inv_freq.data_ptr() if pos is not None else None,
                            c.page_table.stride(0), pos.style if pos is not None else 0,
                            self.nh, self.nkv, self.hd)
        if not self.matmul(xn, self.w_qkv, qkv, ops.MODE_STORE_F32, rope=rope):
            rt.ops.rope_cache_write(
                qkv, q, c.k_pages if self.own_cache else None, c.v_pages if self.own_cache else None,
                batch.token_pos, batch.token_seq, batch.seq_slot,
                c.page_table if self.own_cache else None,
                pos.inv_freq if pos is not None else None, pos.style if pos is not None else 0,
                self.nh, self.nkv, self.hd)
        out = ws.get("attn_out", (T, self.nh * self.hd), rt.act_dtype)
        done = False
        if self.fast is not None:
            done = self.fast.run(q, c, out, batch, self.nh, self.nkv, self.window, self.scale, ws)
        if not done:
            rt.ops.attn_generic(q, c.k_pages, c.v_pages, out, batch.token_pos, batch.token_seq,
                                batch.seq_slot, c.page_table, self.nh, self.nkv, self.hd,
                                self.window, self.scale)
        self.matmul(out, self.w_o, residual, ops.MODE_ACCUM_F32, emit=emit)
