"""An architecture that exists only in this file: its configuration class, its tensor names
(`wte`, `wpe`, `h.<i>.ln_1`, `h.<i>.attn.*`, `h.<i>.ln_post`, `h.<i>.ln_2`, `h.<i>.ffn.*`,
`ln_f`; the head is the embedding table), a block kind with three norms, an embedding multiplier, a
learned position table and a soft cap of the logits.  It is registered, written as a model folder, loaded
through the package's entry point and stepped, with no change to the package's files, and
compared with the same arrangement put together from the plain parts.  It is a toy for the
interfaces; it is nobody's model."""
import math
from dataclasses import dataclass

import numpy as np
import pytest
import torch

from plain import mistral_plain as plain
from tiny import read_weights_numpy

pytestmark = pytest.mark.gpu

ARCH = "ToyDecoderForTests"


def _register():
    import torchless_rs_b200 as tl
    from torchless_rs_b200.config import LayerSpec, ModelSpec, PartSpec
    from torchless_rs_b200.config.reader import KeyReader
    from torchless_rs_b200.parts import register_block

    @register_block("toy_sandwich")
    class SandwichBlock:
        """h += post_norm(mixer(norm_1(h))); h += feed_forward(norm_2(h)).  It has the plain
        block interface only (no carry)."""
        norm_roles = ("mixer_norm", "mixer_post_norm", "feed_forward_norm")

        def __init__(self, spec, rt, mixer, feed_forward, norms):
            self.rt, self.mixer, self.feed_forward, self.norms = rt, mixer, feed_forward, dict(norms)

        def forward(self, x, batch):
            rt = self.rt
            xn = rt.workspace.get("toy_normed", x.shape, rt.act_dtype)
            branch = rt.workspace.get("toy_branch", x.shape, torch.float32)
            branch.zero_()
            self.mixer.forward(self.norms["mixer_norm"](x, xn), branch, batch)
            x += self.norms["mixer_post_norm"](branch, xn).float()
            self.feed_forward.forward(self.norms["feed_forward_norm"](x, xn), x, batch)

    @tl.register_architecture(ARCH)
    @dataclass(frozen=True)
    class ToyConfig:
        n_layer: int
        n_embd: int
        n_head: int
        n_kv: int
        d_head: int
        n_inner: int
        n_vocab: int
        n_pos: int
        eps: float
        theta: float
        cap: float

        @classmethod
        def from_dict(cls, data, where="config.json"):
            r = KeyReader(data, where)
            return cls(r.integer("n_layer"), r.integer("n_embd"), r.integer("n_head"), r.integer("n_kv"),
                       r.integer("d_head"), r.integer("n_inner"), r.integer("n_vocab"), r.integer("n_pos"),
                       r.number("eps"), r.number("theta"), r.number("cap"))

        def to_dict(self):
            d = dict(self.__dict__)
            d["architectures"] = [ARCH]
            return d

        max_position_embeddings = 512

        def model_spec(self):
            norm = PartSpec("rmsnorm", {"size": self.n_embd, "eps": self.eps})
            names = {"mixer_norm": "ln_1", "mixer": "attn", "mixer_post_norm": "ln_post",
                     "feed_forward_norm": "ln_2", "feed_forward": "ffn"}
            layers = tuple(
                LayerSpec(prefix=f"h.{i}", block=PartSpec("toy_sandwich"),
                          mixer=PartSpec("attention", {"hidden_size": self.n_embd, "num_heads": self.n_head,
                                                       "num_kv_heads": self.n_kv, "head_dim": self.d_head,
                                                       "window": None}),
                          feed_forward=PartSpec("swiglu", {"hidden_size": self.n_embd,
                                                           "intermediate_size": self.n_inner}),
                          norms={"mixer_norm": norm, "mixer_post_norm": norm, "feed_forward_norm": norm},
                          names=names,
                          position=PartSpec("rope_half_split", {"head_dim": self.d_head, "theta": self.theta}))
                for i in range(self.n_layer))
            return ModelSpec(hidden_size=self.n_embd, vocab_size=self.n_vocab, embedding_name="wte.weight",
                             head_name="out.weight", tie_head_to_embedding=True, final_norm=norm,
                             final_norm_prefix="ln_f", layers=layers, order=tuple(range(self.n_layer)),
                             embedding_scale=math.sqrt(self.n_embd), position_table_name="wpe.weight",
                             max_positions=self.n_pos, logit_softcap=self.cap)
    return ToyConfig


CFG = dict(architectures=[ARCH], n_layer=2, n_embd=128, n_head=4, n_kv=2, d_head=64, n_inner=320, n_vocab=300,
           n_pos=160, eps=1e-5, theta=1e4, cap=0.25)


def _plain_logits(w, toks):
    n = len(toks)
    pos = np.arange(n)
    h = plain.embedding(w["wte.weight"], toks) * np.float32(math.sqrt(CFG["n_embd"])) + w["wpe.weight"][pos]
    for i in range(CFG["n_layer"]):
        lw = {k[len(f"h.{i}."):]: v for k, v in w.items() if k.startswith(f"h.{i}.")}
        a, _ = plain.attention_mixer(plain.rmsnorm(h, lw["ln_1.weight"], CFG["eps"]), lw["attn.q_proj.weight"],
                                     lw["attn.k_proj.weight"], lw["attn.v_proj.weight"], lw["attn.o_proj.weight"],
                                     pos, CFG["n_head"], CFG["n_kv"], CFG["d_head"], CFG["theta"], None)
        h = h + plain.rmsnorm(a, lw["ln_post.weight"], CFG["eps"])
        h = h + plain.swiglu(plain.rmsnorm(h, lw["ln_2.weight"], CFG["eps"]), lw["ffn.gate_proj.weight"],
                             lw["ffn.up_proj.weight"], lw["ffn.down_proj.weight"])
    logits = plain.rmsnorm(h, w["ln_f.weight"], CFG["eps"]) @ w["wte.weight"].T      # the head is tied
    return CFG["cap"] * np.tanh(logits / CFG["cap"])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_an_architecture_defined_outside_the_package(dtype, tmp_path):
    import torchless_rs_b200 as tl
    from torchless_rs_b200.cache import CacheCapacityError
    _register()
    cfg = tl.config_from_dict(CFG)
    store = torch.float32 if dtype == "float32" else torch.bfloat16
    d = tl.write_random_model(cfg, str(tmp_path), 17, store)
    w = read_weights_numpy(d)
    assert "h.1.attn.k_proj.weight" in w and "h.0.ln_post.weight" in w and "wpe.weight" in w
    assert "out.weight" not in w, "a tied head has no tensor of its own"
    m = tl.load(d, dtype=dtype, max_tokens=512)
    assert type(m.config).__name__ == "ToyConfig"
    rng = np.random.default_rng(5)
    reqs = [[int(t) for t in rng.integers(0, CFG["n_vocab"], n)] for n in (90, 33)]
    slots = m.start_sequences(2)
    pre = [70, 20]
    out = m.step(slots, [r[:p] for r, p in zip(reqs, pre)], "all").cpu().numpy().copy()
    got = [[out[:70]], [out[70:]]]
    fed, live = list(pre), [0, 1]
    while live:
        out = m.step([slots[i] for i in live], [[reqs[i][fed[i]]] for i in live], "last").cpu().numpy().copy()
        for j, i in enumerate(live):
            got[i].append(out[j:j + 1]); fed[i] += 1
        done = [i for i in live if fed[i] >= len(reqs[i])]
        m.end_sequences([slots[i] for i in done])
        live = [i for i in live if i not in done]
    for i, r in enumerate(reqs):
        ref, g = _plain_logits(w, r), np.concatenate(got[i])
        assert np.abs(ref).max() > 0.6 * CFG["cap"], "the cap does not bend these logits: the test shows nothing"
        bound = 5e-5 + 1e-4 * np.abs(ref) if dtype == "float32" else 2.5e-2 * np.abs(ref).max()
        assert (np.abs(g - ref) <= bound).all(), f"request {i}: max err {np.abs(g - ref).max():.3e}"
    # the position table has 160 rows: a longer sequence is refused before anything runs
    (s,) = m.start_sequences(1)
    with pytest.raises(CacheCapacityError):
        m.step([s], [[1] * 161], "last")
    m.end_sequences([s])
    m.engine.cache.check()
