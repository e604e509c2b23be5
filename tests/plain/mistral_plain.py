"""Plain, slow restatement of the Mistral dense decoder, for tests only.

It rests on the formulas of rglonek/torchless-rs (file:line cited at each
function, paths inside that project).  The reference's own model code is Rust
and no Rust toolchain exists where these tests run, so nothing here was checked
against a run of the reference: it rests on the formulas alone.

Whole sequences, no cache, one function per part, numpy only.  It shares no
code with the package under test.  `dtype` is numpy float32 by default;
float64 gives a higher-precision oracle for error-budget checks.
"""
from __future__ import annotations

import math

import numpy as np


def embedding(table: np.ndarray, tokens) -> np.ndarray:
    """h <- E[token, :], no scaling.  src/model/modules/embedding.rs:15-21."""
    return table[np.asarray(tokens, dtype=np.int64)]


def rmsnorm(x: np.ndarray, weight: np.ndarray, eps: float) -> np.ndarray:
    """y = x / sqrt(mean(x^2) + eps) * w; the weight is used as it is.
    src/kernels/mod.rs:558-568."""
    ss = np.sum(x * x, axis=-1, keepdims=True)
    rms = np.sqrt(ss / x.shape[-1] + x.dtype.type(eps))
    return (x / rms) * weight


def rope_inv_freq(head_dim: int, theta: float, dtype=np.float32) -> np.ndarray:
    """inv_freq[i] = 1 / theta^(i / (head_dim/2)), i in [0, head_dim/2).
    src/kernels/mod.rs:572-580."""
    half = head_dim // 2
    i = np.arange(half, dtype=np.float64)
    return (1.0 / np.power(float(theta), i / half)).astype(dtype)


def rope_cos_sin(inv_freq: np.ndarray, positions) -> tuple[np.ndarray, np.ndarray]:
    """angle = inv_freq * pos; cos and sin of it.  src/kernels/mod.rs:583-588."""
    pos = np.asarray(positions, dtype=inv_freq.dtype)[:, None]
    ang = pos * inv_freq[None, :]
    return np.cos(ang), np.sin(ang)


def apply_rope(x: np.ndarray, cos: np.ndarray, sin: np.ndarray) -> np.ndarray:
    """Half-split pairing: dimension i turns with dimension i + head_dim/2.
    x: [n, heads, head_dim]; cos, sin: [n, head_dim/2].
    src/kernels/mod.rs:590-608."""
    half = x.shape[-1] // 2
    a, b = x[..., :half], x[..., half:]
    c, s = cos[:, None, :], sin[:, None, :]
    return np.concatenate([a * c - b * s, a * s + b * c], axis=-1)


def softmax(s: np.ndarray) -> np.ndarray:
    """Max-subtracted softmax over the last axis.  src/kernels/mod.rs:529-543."""
    m = np.max(s, axis=-1, keepdims=True)
    e = np.exp(s - m)
    return e / np.sum(e, axis=-1, keepdims=True)


def attention_scores_mask(n: int, window) -> np.ndarray:
    """Boolean [n, n], True where query p may see key i: i <= p (only 0..=p exist,
    src/model/modules/attention.rs:88-105) and, with a window W, not
    (p >= W and i < p - W + 1), i.e. i in [p-W+1, p]
    (the inequality of src/model/models/gpt_oss.rs:168-176)."""
    p = np.arange(n)[:, None]
    i = np.arange(n)[None, :]
    ok = i <= p
    if window:
        ok &= ~((p >= window) & (i < p - window + 1))
    return ok


def attention(q: np.ndarray, k: np.ndarray, v: np.ndarray, window) -> np.ndarray:
    """Grouped-query attention of one whole sequence.
    q: [n, nh, hd]; k, v: [n, nkv, hd] (k already rotated).  Query head h reads
    key/value head h // (nh/nkv); scores scaled by 1/sqrt(hd); softmax; weighted
    sum of values.  src/model/modules/attention.rs:78-121."""
    n, nh, hd = q.shape
    nkv = k.shape[1]
    group = nh // nkv
    scale = q.dtype.type(1.0 / math.sqrt(hd))
    ok = attention_scores_mask(n, window)
    out = np.empty_like(q)
    for h in range(nh):
        kvh = h // group
        s = (q[:, h, :] @ k[:, kvh, :].T) * scale
        s = np.where(ok, s, -np.inf).astype(q.dtype)
        p = softmax(s)
        out[:, h, :] = p @ v[:, kvh, :]
    return out


def attention_mixer(x, wq, wk, wv, wo, positions, nh, nkv, hd, theta, window,
                    kv_override=None):
    """q/k/v projections without bias, rotation of q and k at each token's
    position, attention, output projection over the head-major concatenation.
    src/model/modules/attention.rs:46-135.  `kv_override` = (k, v) of another
    layer, for a layer that reads another layer's cache (then wk and wv are unused).
    Returns (out, (k, v))."""
    n = x.shape[0]
    inv = rope_inv_freq(hd, theta, x.dtype)
    cos, sin = rope_cos_sin(inv, positions)
    q = apply_rope((x @ wq.T).reshape(n, nh, hd), cos, sin)
    if kv_override is None:
        k = apply_rope((x @ wk.T).reshape(n, nkv, hd), cos, sin)
        v = (x @ wv.T).reshape(n, nkv, hd)
    else:
        k, v = kv_override
    ctx = attention(q, k, v, window)
    return ctx.reshape(n, nh * hd) @ wo.T, (k, v)


def silu(z: np.ndarray) -> np.ndarray:
    """z / (1 + exp(-z)).  src/kernels/mod.rs:546-548."""
    return z / (1.0 + np.exp(-z))


def swiglu(x, w_gate, w_up, w_down) -> np.ndarray:
    """down( silu(gate x) * (up x) ).  src/model/modules/mlp.rs:23-45."""
    return (silu(x @ w_gate.T) * (x @ w_up.T)) @ w_down.T


def block(h, lw, positions, cfg, window):
    """Pre-norm residual block: h += Attn(Norm1(h)); h += MLP(Norm2(h)); the
    residual is the stream before the norm.  src/model/modules/layer.rs:28-56."""
    a, _ = attention_mixer(
        rmsnorm(h, lw["input_layernorm.weight"], cfg["rms_norm_eps"]),
        lw["self_attn.q_proj.weight"], lw["self_attn.k_proj.weight"],
        lw["self_attn.v_proj.weight"], lw["self_attn.o_proj.weight"],
        positions, cfg["num_attention_heads"], cfg["num_key_value_heads"],
        cfg["head_dim"], cfg["rope_theta"], window)
    h = h + a
    m = swiglu(rmsnorm(h, lw["post_attention_layernorm.weight"], cfg["rms_norm_eps"]),
               lw["mlp.gate_proj.weight"], lw["mlp.up_proj.weight"],
               lw["mlp.down_proj.weight"])
    return h + m


def normalise_config(cfg: dict) -> dict:
    """Defaults the reference uses: KV heads = heads
    (src/loader/formats/safetensors.rs:731-735), rope_theta 10000 and eps 1e-5
    (src/loader/formats/gguf.rs:1200-1202), head_dim = hidden/heads
    (src/model/mod.rs:143) unless config.json gives one."""
    c = dict(cfg)
    c.setdefault("num_key_value_heads", c["num_attention_heads"])
    c.setdefault("rope_theta", 10000.0)
    c.setdefault("rms_norm_eps", 1e-5)
    if not c.get("head_dim"):
        c["head_dim"] = c["hidden_size"] // c["num_attention_heads"]
    c.setdefault("sliding_window", None)
    return c


def forward_logits(cfg: dict, weights: dict, tokens, dtype=np.float32) -> np.ndarray:
    """Logits [n, vocab] at every position of one whole sequence that starts at
    position 0: embed, the blocks in order, final norm, untied LM head.
    src/model/mod.rs:430-447.  `weights` maps the tensor names of
    src/model/mod.rs:360-414 to arrays."""
    cfg = normalise_config(cfg)
    w = {k: np.asarray(v, dtype=dtype) for k, v in weights.items()}
    n = len(tokens)
    positions = np.arange(n)
    h = embedding(w["model.embed_tokens.weight"], tokens)
    for layer in range(cfg["num_hidden_layers"]):
        pre = f"model.layers.{layer}."
        lw = {k[len(pre):]: v for k, v in w.items() if k.startswith(pre)}
        h = block(h, lw, positions, cfg, cfg["sliding_window"])
    h = rmsnorm(h, w["model.norm.weight"], cfg["rms_norm_eps"])
    return h @ w["lm_head.weight"].T


# ---------------------------------------------------------------------------
# Sampling (src/sampler/mod.rs)
# ---------------------------------------------------------------------------

def greedy(logits: np.ndarray) -> int:
    """Arg-max of the logits; on an exact tie the last maximal index, as Rust's
    `max_by` returns it.  src/sampler/mod.rs:60-68."""
    n = len(logits)
    return int(n - 1 - np.argmax(np.asarray(logits)[::-1]))


def top_k_filter(scaled: np.ndarray, k: int) -> np.ndarray:
    """Keep the k largest of the temperature-scaled logits, the rest become -inf;
    on ties at the threshold keep the first ones in index order until k are kept.
    src/sampler/mod.rs:93-119."""
    out = scaled.copy()
    thr = np.sort(scaled)[::-1][min(k, len(scaled)) - 1]
    if np.count_nonzero(scaled >= thr) <= k:
        out[scaled < thr] = -np.inf
        return out
    kept = 0
    for i in range(len(out)):
        if out[i] >= thr and kept < k:
            kept += 1
        else:
            out[i] = -np.inf
    return out


def top_p_filter(probs: np.ndarray, p: float) -> np.ndarray:
    """Sort descending, keep the shortest prefix whose sum is >= p, zero the rest,
    renormalise.  src/sampler/mod.rs:144-170."""
    order = np.argsort(-probs, kind="stable")
    csum = np.cumsum(probs[order])
    cutoff = int(np.searchsorted(csum, p, side="left")) + 1
    out = np.zeros_like(probs)
    keep = order[:cutoff]
    out[keep] = probs[keep]
    return out / out.sum()


def sample_probs(logits: np.ndarray, temperature: float, top_k=None, top_p=None) -> np.ndarray:
    """The distribution the reference draws from: logits / T, top-k, softmax,
    top-p.  src/sampler/mod.rs:194-222."""
    z = logits.astype(np.float64) / temperature
    if top_k and 0 < top_k < len(z):
        z = top_k_filter(z, top_k)
    pr = softmax(z)
    if top_p and 0.0 < top_p < 1.0:
        pr = top_p_filter(pr, top_p)
    return pr


def draw(probs: np.ndarray, r: float) -> int:
    """Inverse CDF: the first index whose running sum is >= r, else the last.
    src/sampler/mod.rs:225-238."""
    c = np.cumsum(probs)
    idx = int(np.searchsorted(c, r, side="left"))
    return min(idx, len(probs) - 1)
