"""The plain implementation checked against itself and against hand-made cases (no
device needed): it is the oracle of the GPU tests, so its parts are pinned here."""
import os

import numpy as np

from plain import mistral_plain as plain
from tiny import CONFIGS, make_model_dir, read_weights_numpy


def test_rmsnorm_by_hand():
    x = np.array([[3.0, 4.0]], dtype=np.float32)
    y = plain.rmsnorm(x, np.array([2.0, 0.5], dtype=np.float32), 0.0)
    rms = np.sqrt(12.5)
    assert np.allclose(y, [[3 / rms * 2, 4 / rms * 0.5]])


def test_rope_properties():
    inv = plain.rope_inv_freq(8, 10000.0)
    assert inv[0] == 1.0 and np.all(np.diff(inv) < 0)                 # reference: kernels/tests.rs:53-69
    cos, sin = plain.rope_cos_sin(inv, [0, 3])
    assert np.allclose(cos[0], 1) and np.allclose(sin[0], 0)          # kernels/tests.rs:71-84
    x = np.arange(16, dtype=np.float32).reshape(1, 2, 8)
    y = plain.apply_rope(np.repeat(x, 2, 0), cos, sin)
    assert np.allclose(y[0], x[0])                                    # position 0 changes nothing
    assert np.allclose(np.linalg.norm(y[1], axis=-1), np.linalg.norm(x[0], axis=-1), rtol=1e-5)
    # half-split pairing: dimension 0 turns with dimension 4 by angle 3 * inv[0]
    a, b = x[0, 0, 0], x[0, 0, 4]
    assert np.isclose(y[1, 0, 0], a * np.cos(3.0) - b * np.sin(3.0), rtol=1e-5)


def test_window_mask_edges():
    ok = plain.attention_scores_mask(6, 3)
    assert ok[5].tolist() == [False, False, False, True, True, True]   # keys p-W+1 .. p
    assert ok[2].tolist() == [True, True, True, False, False, False]
    assert plain.attention_scores_mask(4, None)[3].tolist() == [True] * 4


def test_attention_is_causal_and_grouped():
    rng = np.random.default_rng(0)
    q = rng.standard_normal((5, 4, 8)).astype(np.float32)
    k = rng.standard_normal((5, 2, 8)).astype(np.float32)
    v = rng.standard_normal((5, 2, 8)).astype(np.float32)
    out = plain.attention(q, k, v, None)
    assert np.allclose(out[0, 0], v[0, 0]) and np.allclose(out[0, 3], v[0, 1])   # first token sees itself only
    k2, v2 = k.copy(), v.copy()
    k2[4], v2[4] = 9.0, 9.0
    assert np.allclose(plain.attention(q, k2, v2, None)[:4], out[:4])           # the future changes nothing


def test_float32_agrees_with_float64_on_a_tiny_model():
    cfg = CONFIGS["B"]
    w = read_weights_numpy(make_model_dir(cfg, 1))
    toks = [int(t) for t in np.random.default_rng(1).integers(0, cfg["vocab_size"], 40)]
    a = plain.forward_logits(cfg, w, toks, np.float32)
    b = plain.forward_logits(cfg, w, toks, np.float64)
    assert a.shape == (40, cfg["vocab_size"]) and np.abs(a - b).max() < 2e-5
    # a prefix gives the same logits: no position looks ahead
    assert np.abs(plain.forward_logits(cfg, w, toks[:17], np.float64) - b[:17]).max() < 1e-12


def test_window_changes_logits_only_beyond_the_window():
    cfg = dict(CONFIGS["A"])
    w = read_weights_numpy(make_model_dir(cfg, 2))
    toks = [int(t) for t in np.random.default_rng(2).integers(0, 256, 30)]
    with_w = plain.forward_logits(cfg, w, toks, np.float64)
    cfg["sliding_window"] = None
    without = plain.forward_logits(cfg, w, toks, np.float64)
    assert np.abs(with_w[:16] - without[:16]).max() < 1e-12
    assert np.abs(with_w[16:] - without[16:]).max() > 1e-6


def test_sampling_parts():
    logits = np.array([0.1, 2.0, -1.0, 2.0, 0.5], dtype=np.float32)
    assert plain.greedy(np.array([0.1, 2.0, -1.0, 1.9])) == 1              # sampler/tests.rs:34-50
    assert plain.greedy(np.array([3.0, 1.0, 3.0])) == 2                    # Rust's max_by keeps the last of equal maxima
    f = plain.top_k_filter(logits.astype(np.float64), 1)
    assert np.isfinite(f).sum() == 1 and np.isfinite(f[1])                  # ties: first in index order
    p = plain.sample_probs(logits, 0.7)
    assert np.isclose(p.sum(), 1.0)                                         # sampler/tests.rs:69-90
    hot, cold = plain.sample_probs(logits, 2.0), plain.sample_probs(logits, 0.5)
    assert hot.max() < cold.max()                                           # sampler/tests.rs:92-134
    assert np.count_nonzero(plain.sample_probs(logits, 1.0, top_k=2)) == 2  # sampler/tests.rs:183-203
    assert np.allclose(plain.sample_probs(logits, 1.0, top_k=9), plain.sample_probs(logits, 1.0))
    pp = plain.sample_probs(logits, 1.0, top_p=0.5)
    assert np.isclose(pp.sum(), 1.0) and np.count_nonzero(pp) == 2
    assert plain.draw(np.array([0.2, 0.3, 0.5]), 0.25) == 1 and plain.draw(np.array([0.2, 0.3, 0.5]), 0.99) == 2


def test_two_independent_restatements_agree(tmp_path):
    """The numpy restatement (whole sequences, matrix products, no cache) and the C++ one
    (one token per forward pass with a cache, sequential dot products, the reference's own
    shape of the computation) agree to rounding on three configurations, two of them with a
    window shorter than the sequence, from bfloat16, float16 and 32-bit folders.  The
    reference checks one implementation against another in the same way
    (src/model/modules/tests.rs:213-245, at 1e-4)."""
    import subprocess
    import torch
    from tiny import make_model_dir, read_weights_numpy
    src = os.path.join(os.path.dirname(__file__), "plain", "mistral_plain_onetoken.cpp")
    exe = str(tmp_path / "mistral_plain_onetoken")
    subprocess.run(["g++", "-O2", "-std=c++17", "-o", exe, src], check=True)
    for name, store in (("A", torch.float32), ("B", torch.bfloat16), ("C", torch.float16)):
        cfg = CONFIGS[name]
        d = make_model_dir(cfg, 5, store, str(tmp_path / name))
        toks = [int(t) for t in np.random.default_rng(1).integers(0, cfg["vocab_size"], 90)]
        with open(os.path.join(d, "tokens.txt"), "w") as f:
            f.write(" ".join(map(str, toks)))
        subprocess.run([exe, d, os.path.join(d, "tokens.txt"), os.path.join(d, "logits.f32")], check=True)
        got = np.fromfile(os.path.join(d, "logits.f32"), dtype=np.float32).reshape(len(toks), -1)
        ref = plain.forward_logits(cfg, read_weights_numpy(d), toks)
        assert np.abs(got - ref).max() <= 1e-5, f"configuration {name}: {np.abs(got - ref).max():.3e}"
