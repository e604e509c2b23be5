"""Configurations drawn at random from what config.json allows (head sizes in steps of 16, any
number of heads and groups, widths and vocabularies that are no powers of two, with and without
a window, narrow and wide enough for the split-K products), each run as an unequal batch that
starts together and then decodes token by token, against the plain implementation.  The seeds
are fixed; each case draws its sizes, its type and its batch from its seed."""
import random

import numpy as np
import pytest
import torch

from helpers_gpu import TinyModel, assert_close

pytestmark = pytest.mark.gpu


def _draw(seed: int):
    rnd = random.Random(seed)
    wide = seed % 2 == 1
    hd = rnd.choice([16, 32, 48, 64, 64, 128, 128, 80, 256])
    nkv = rnd.choice([1, 2, 3, 4])
    nh = nkv * rnd.choice([1, 2, 3, 4, 8, 12])
    limit = 4096 if wide else 2048
    if nh * hd > limit:
        nh = max(nkv, (limit // hd) // nkv * nkv)
    if nh < nkv:
        nkv = nh = 1
    cfg = dict(architectures=["MistralForCausalLM"], model_type="mistral",
               num_hidden_layers=rnd.choice([1, 2, 3]),
               hidden_size=rnd.choice([512, 640, 768, 1024, 520] if wide else [64, 72, 96, 100, 128, 136, 84]),
               num_attention_heads=nh, num_key_value_heads=nkv, head_dim=hd,
               intermediate_size=rnd.choice([1024, 1416, 2048, 2816] if wide else [96, 100, 176, 200, 328]),
               vocab_size=rnd.choice([97, 256, 331, 1000]), rope_theta=rnd.choice([1e4, 1e6]),
               sliding_window=rnd.choice([None, None, 7, 33, 64, 100, 129]),
               rms_norm_eps=rnd.choice([1e-5, 1e-6]), tie_word_embeddings=False, max_position_embeddings=4096)
    dtype = rnd.choice(["float32", "bfloat16", "bfloat16"])
    batch = rnd.choice([1, 2, 3, 5, 9, 17])
    return cfg, dtype, batch


@pytest.mark.parametrize("seed", [7001, 7002, 7003, 7004, 7005, 7006, 7007, 7008, 7010, 7011, 7013, 7016])
def test_a_drawn_configuration(seed):
    cfg, dtype, B = _draw(seed)
    tm = TinyModel("drawn", dtype, seed=seed, max_tokens=4096, cfg=cfg)
    rng = np.random.default_rng(seed)
    lens = [int(rng.integers(1, 300 if B <= 3 else 70)) for _ in range(B)]
    reqs = [[int(t) for t in rng.integers(0, cfg["vocab_size"], n)] for n in lens]
    pre = [int(rng.integers(1, n + 1)) for n in lens]
    slots = tm.engine.start_sequences(B)
    out = tm.step_np(slots, [r[:p] for r, p in zip(reqs, pre)], "all")
    got, o = [[] for _ in reqs], 0
    for i, p in enumerate(pre):
        got[i].append(out[o:o + p]); o += p
    fed, live = list(pre), list(range(B))
    while True:
        done = [i for i in live if fed[i] >= len(reqs[i])]
        if done:
            tm.engine.end_sequences([slots[i] for i in done])
            live = [i for i in live if i not in done]
        if not live:
            break
        out = tm.step_np([slots[i] for i in live], [[reqs[i][fed[i]]] for i in live], "last")
        for j, i in enumerate(live):
            got[i].append(out[j:j + 1]); fed[i] += 1
    what = {k: cfg[k] for k in ("hidden_size", "num_attention_heads", "num_key_value_heads", "head_dim",
                                "intermediate_size", "vocab_size", "sliding_window", "num_hidden_layers")}
    for i, r in enumerate(reqs):
        assert_close(np.concatenate(got[i]), tm.reference(r), dtype, f"{what} {dtype} request {i} n={len(r)} pre={pre[i]}")
    tm.engine.cache.check()
    tm.engine.check_kernels()
