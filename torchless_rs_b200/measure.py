"""Single-kernel runs for timing and profiling.

    python -m torchless_rs_b200.measure gemm M N K MODE [--iters I]
    python -m torchless_rs_b200.measure attn-decode BATCH CONTEXT [--iters I]
    python -m torchless_rs_b200.measure attn-prefill TOKENS [--iters I]
    python -m torchless_rs_b200.measure elementwise TOKENS [--iters I]
    python -m torchless_rs_b200.measure step BATCH CONTEXT PREFILL_TOKENS [--layers L] [--iters I]
    python -m torchless_rs_b200.measure timeline BATCH CONTEXT [--layers L]

Each prints the mean device time per launch (CUDA events, after warm-up; the weights
or the cache are larger than the L2 cache or rotated so that they come from HBM) and
the bandwidth or arithmetic rate that this time means.  Sizes other than the ones
given default to those of Mistral 7B (32 heads, 8 key/value heads, head size 128).

`step` runs whole steps of the engine, kernel by kernel (no CUDA graph), on a model with
the layer sizes of Mistral 7B, random weights and L layers: I prefill steps of
PREFILL_TOKENS tokens, then I decode steps of BATCH sequences that hold CONTEXT tokens of
random cache content.  It is the small case for a profiler's list of launches: which kernels
a step consists of and how its time divides among them.
"""
from __future__ import annotations

import argparse
import math

import torch


def _time(fn, iters: int) -> float:
    """Mean microseconds per call.  The calls are recorded into one CUDA graph and the graph
    is replayed, so the host's launch cost (some ten microseconds per call from Python) does
    not bound what is measured."""
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for _ in range(iters):
            fn()
    graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(3):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / (3 * iters)   # microseconds


def gemm(M: int, N: int, K: int, mode: int, iters: int) -> None:
    from .csrc.gemm_bf16 import GemmBf16
    g = GemmBf16.get()
    rows = 2 * N if mode == 2 else N
    copies = max(2, int(400e6 // (rows * K * 2)) + 1)     # rotate weights: more than the L2 holds
    ws = [torch.randn((rows, K), device="cuda", dtype=torch.bfloat16) * 0.02 for _ in range(copies)]
    x = torch.randn((M, K), device="cuda", dtype=torch.bfloat16)
    out = torch.zeros((M, N), device="cuda", dtype=torch.float32 if mode in (0, 1) else torch.bfloat16)
    state = {"i": 0}

    def run():
        assert g.run(x, ws[state["i"] % copies], out, mode), "shape not taken by the tensor-core kernel"
        state["i"] += 1
    us = _time(run, iters)
    print(f"gemm M={M} N={N} K={K} mode={mode}: {us:.2f} us, "
          f"{rows * K * 2 / us / 1e3:.0f} GB/s of weights, {2.0 * M * rows * K / us / 1e6:.1f} TFLOP/s, "
          f"error word {g.take_error()}")


def _paged(B: int, ctx: int, nkv: int, hd: int):
    pages = (ctx + 63) // 64
    kp = torch.randn((B * pages, nkv, 64, hd), device="cuda", dtype=torch.bfloat16)
    vp = torch.randn((B * pages, nkv, hd, 64), device="cuda", dtype=torch.bfloat16)
    table = torch.arange(B * pages, dtype=torch.int32, device="cuda").view(B, pages)
    slot = torch.arange(B, dtype=torch.int32, device="cuda")
    return kp, vp, table, slot


def attn_decode(B: int, ctx: int, iters: int, nh=32, nkv=8, hd=128) -> None:
    from .csrc import attention_bf16
    from .csrc.attention_bf16 import AttentionBf16
    from .parts.runtime import Workspace
    decode_splits = attention_bf16.decode_splits
    att, ws = AttentionBf16.get(hd), Workspace(torch.device("cuda"))
    kp, vp, table, slot = _paged(B, ctx, nkv, hd)
    lens = torch.full((B,), ctx, dtype=torch.int32, device="cuda")
    q = torch.randn((B, nh * hd), device="cuda", dtype=torch.bfloat16)
    out = torch.empty_like(q)
    n = decode_splits(B, nkv, ctx, None)
    us = _time(lambda: att.decode(q, kp, vp, out, lens, slot, table, nh, nkv, None,
                                  1 / math.sqrt(hd), n, ws), iters)
    byts = 2.0 * B * ctx * nkv * hd * 2
    print(f"attn-decode B={B} context={ctx} splits={n}: {us:.2f} us (both kernels), {byts / us / 1e3:.0f} GB/s of cache")


def attn_prefill(T: int, iters: int, nh=32, nkv=8, hd=128) -> None:
    from .csrc.attention_bf16 import AttentionBf16
    att = AttentionBf16.get(hd)
    kp, vp, table, slot = _paged(1, T, nkv, hd)
    start = torch.tensor([0, T], dtype=torch.int32, device="cuda")
    lens = torch.tensor([T], dtype=torch.int32, device="cuda")
    q = torch.randn((T, nh * hd), device="cuda", dtype=torch.bfloat16)
    out = torch.empty_like(q)
    for variant in ("tc", "tma"):
        us = _time(lambda: att.prefill(q, kp, vp, out, start, lens, slot, table, 1, T, nh, nkv, None,
                                       1 / math.sqrt(hd), variant=variant), iters)
        print(f"attn-prefill tokens={T} kernel={variant}: {us:.2f} us, "
              f"{2.0 * nh * hd * T * T / us / 1e6:.1f} TFLOP/s (causal half counted), error word {att.take_error()}")


def elementwise(T: int, iters: int, H=4096, nh=32, nkv=8, hd=128) -> None:
    """The norm kernel and the rotation + cache write kernel of a prefill step of T tokens, each with inputs
    rotated through more than the L2 cache holds and with one input over and over (as in a step, where the
    kernel before has just written it)."""
    from .csrc import ops
    o = ops.core_ops(torch.bfloat16)
    copies = max(2, int(400e6 // (T * H * 4)) + 1)
    xs = [torch.randn((T, H), device="cuda") for _ in range(copies)]
    w = torch.ones(H, device="cuda", dtype=torch.bfloat16)
    y = torch.empty((T, H), device="cuda", dtype=torch.bfloat16)
    st = {"i": 0}

    def norm(rotate):
        o.rmsnorm(xs[st["i"] % copies if rotate else 0], w, 1e-5, y)
        st["i"] += 1
    byts = T * H * 6.0
    for rotate in (True, False):
        us = _time(lambda: norm(rotate), iters)
        print(f"rmsnorm {T} x {H}, {'inputs from HBM' if rotate else 'input in L2'}: {us:.2f} us, {byts / us / 1e3:.0f} GB/s")
    cols = (nh + 2 * nkv) * hd
    copies = max(2, int(400e6 // (T * cols * 4)) + 1)
    qkvs = [torch.randn((T, cols), device="cuda") for _ in range(copies)]
    q = torch.empty((T, nh * hd), device="cuda", dtype=torch.bfloat16)
    pages = (T + 63) // 64
    kp = torch.zeros((pages, nkv, 64, hd), device="cuda", dtype=torch.bfloat16)
    vp = torch.zeros((pages, nkv, hd, 64), device="cuda", dtype=torch.bfloat16)
    pos = torch.arange(T, dtype=torch.int32, device="cuda")
    seq = torch.zeros(T, dtype=torch.int32, device="cuda")
    slot = torch.zeros(1, dtype=torch.int32, device="cuda")
    table = torch.arange(pages, dtype=torch.int32, device="cuda").view(1, pages)
    half = hd // 2
    inv = (1.0 / torch.pow(torch.tensor(1e4, dtype=torch.float64),
                           torch.arange(half, dtype=torch.float64) / half)).float().cuda()

    def rope(rotate):
        o.rope_cache_write(qkvs[st["i"] % copies if rotate else 0], q, kp, vp, pos, seq, slot, table, inv, 0, nh, nkv, hd)
        st["i"] += 1
    byts = T * cols * 6.0
    for rotate in (True, False):
        us = _time(lambda: rope(rotate), iters)
        print(f"rotation + cache write, {T} tokens, {'inputs from HBM' if rotate else 'input in L2'}: {us:.2f} us, "
              f"{byts / us / 1e3:.0f} GB/s")


MISTRAL_7B_SIZES = {
    "architectures": ["MistralForCausalLM"], "model_type": "mistral", "hidden_size": 4096,
    "intermediate_size": 14336, "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128,
    "vocab_size": 32000, "rms_norm_eps": 1e-5, "rope_theta": 10000.0, "sliding_window": 4096,
    "max_position_embeddings": 32768, "hidden_act": "silu", "tie_word_embeddings": False,
    "torch_dtype": "bfloat16",
}
# the layer sizes of the two larger workloads that bench.py names (Mistral NeMo 12B, Mistral Small 22B)
MODEL_SIZES = {
    "mistral7b": MISTRAL_7B_SIZES,
    "nemo12b": dict(MISTRAL_7B_SIZES, hidden_size=5120, vocab_size=131072, rope_theta=1e6, sliding_window=None,
                    max_position_embeddings=131072),
    "small22b": dict(MISTRAL_7B_SIZES, hidden_size=6144, num_attention_heads=48, intermediate_size=16384,
                     vocab_size=32768, rope_theta=1e6, sliding_window=None),
}
SIZES = MISTRAL_7B_SIZES   # what `step` and `timeline` build; --model chooses


def step(B: int, context: int, prefill: int, layers: int, iters: int) -> None:
    from . import from_random
    from .config import config_from_dict
    from .sampling.params import SamplingParams
    cfg = dict(SIZES, num_hidden_layers=layers)
    longest = max(context + iters + 1, prefill)
    model = from_random(config_from_dict(cfg), seed=0, dtype="bfloat16",
                        max_tokens=B * (longest + 64) + prefill + 64, max_batch=B + 1, max_seq_len=longest + 64)
    eng = model.engine
    eng.use_graphs = False
    for g in eng.cache.paged:
        g.storage.normal_(0.0, 0.5)

    def timed(fn):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) * 1e3

    prompt = [[(13 * i + 1) % eng.vocab_size for i in range(prefill)]]
    for i in range(iters):
        (s,) = eng.start_sequences(1)
        us = timed(lambda: eng.step([s], prompt, "last"))
        eng.end_sequences([s])
        print(f"prefill step {i}: {prefill} tokens, {layers} layers, {us:.0f} us")
    slots = eng.start_sequences(B)
    eng.cache.prepare(slots, [context] * B)
    eng.cache.commit(slots, [context] * B)
    toks = [[(7 * i + 3) % eng.vocab_size] for i in range(B)]
    greedy = SamplingParams.greedy()
    for i in range(iters):
        us = timed(lambda: model.sampler.select(eng.step(slots, toks, "last"), greedy))
        print(f"decode step {i}: batch {B}, context {context + i}, {layers} layers, {us:.0f} us "
              f"(launched from Python kernel by kernel: the host's launch cost is in this time)")
    eng.end_sequences(slots)
    eng.check_kernels()


def decode(lengths, layers: int, window, equal_shares: bool) -> None:
    """Decode steps as generation runs them (replayed CUDA graph, tokens fed from the device's own choice)
    for sequences that end at the given lengths: us per step and the share of the copy bandwidth that the
    bytes a step has to read would need.  `equal_shares`: the decode attention without its page quantum."""
    from . import from_random
    from .config import config_from_dict
    from .csrc import attention_bf16
    from .sampling.params import SamplingParams
    cfg = dict(SIZES, num_hidden_layers=layers, sliding_window=window, max_position_embeddings=1 << 20)
    B, steps, warm = len(lengths), 32, 6
    model = from_random(config_from_dict(cfg), seed=0, dtype="bfloat16", max_tokens=sum(n + 128 for n in lengths),
                        max_batch=B, max_seq_len=max(lengths) + 128)
    eng = model.engine
    for g in eng.cache.paged:
        g.storage.normal_(0.0, 0.5)
    if equal_shares:
        plain = attention_bf16.decode_splits
        attention_bf16.decode_plan = lambda *a, **k: (plain(*a[:6]), 0)
    slots = eng.start_sequences(B)
    start = [max(1, n - steps - warm) for n in lengths]
    eng.cache.prepare(slots, start)
    eng.cache.commit(slots, start)
    toks = [[(7 * i + 3) % eng.vocab_size] for i in range(B)]
    greedy = SamplingParams.greedy()
    for _ in range(warm):
        model.sampler.select(eng.step(slots, toks, "last"), greedy)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(steps):
        model.sampler.select(eng.step(slots, toks, "last"), greedy)
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / steps
    c = config_from_dict(cfg)
    per_layer = 2 * c.hidden_size * (c.num_attention_heads + 2 * c.num_key_value_heads) * c.head_dim \
        + 2 * c.hidden_size * c.num_attention_heads * c.head_dim + 2 * 3 * c.hidden_size * c.intermediate_size
    spans = [min(n, window) if window else n for n in lengths]
    byts = layers * per_layer + 2 * c.hidden_size * c.vocab_size \
        + layers * sum(spans) * c.num_key_value_heads * c.head_dim * 4
    eng.end_sequences(slots)
    eng.check_kernels()
    print(f"decode, {B} sequences of {min(lengths)} to {max(lengths)} tokens ({sum(lengths)} in all), {layers} layers + head"
          f"{', equal shares' if equal_shares else ''}: {us:.1f} us per step, {byts / us / 1e3:.0f} GB/s of weights and cache")


TRACE_KINDS = {1: "embed", 2: "rmsnorm", 3: "product", 4: "attention", 5: "attention merge", 6: "argmax"}


def timeline(B: int, context: int, layers: int) -> None:
    """One decode step as the engine runs it (a replayed CUDA graph): when each kernel's first
    block started and its last block ended on the GPU's nanosecond timer, and the gap or overlap
    between neighbours.  Uses the diagnostic build of the kernels."""
    import ctypes
    from .csrc import build
    build.TRACE = True
    from . import from_random
    from .config import config_from_dict
    from .sampling.params import SamplingParams
    cfg = dict(SIZES, num_hidden_layers=layers)
    model = from_random(config_from_dict(cfg), seed=0, dtype="bfloat16", max_tokens=B * (context + 128),
                        max_batch=B, max_seq_len=context + 128)
    eng = model.engine
    for g in eng.cache.paged:
        g.storage.normal_(0.0, 0.5)
    slots = eng.start_sequences(B)
    eng.cache.prepare(slots, [context] * B)
    eng.cache.commit(slots, [context] * B)
    toks = [[(7 * i + 3) % eng.vocab_size] for i in range(B)]
    greedy = SamplingParams.greedy()
    readers = [(build.load_library("core_bf16"), "elementwise"), (build.load_library("gemm_tc"), "gemm_tc"),
               (build.load_library("attn_bf16_hd128"), "attn_tma"), (build.load_library("sampling"), "sampling")]

    def take():
        rows = []
        for lib, name in readers:
            buf = (ctypes.c_ulonglong * (4 * 8192))()
            n = getattr(lib, f"tl_trace_take_{name}")(buf, 8192)
            rows += [tuple(buf[4 * i + j] for j in range(4)) for i in range(max(n, 0))]
        return sorted(rows, key=lambda r: r[1])

    for _ in range(5):      # eager, recorded, then replayed
        model.sampler.select(eng.step(slots, toks, "last"), greedy)
    torch.cuda.synchronize()
    take()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    model.sampler.select(eng.step(slots, toks, "last"), greedy)
    e1.record()
    torch.cuda.synchronize()
    rows = take()
    t0 = rows[0][1]
    print(f"decode step, batch {B}, context {context + 5}, {layers} layers: {e0.elapsed_time(e1) * 1e3:.1f} us by events, "
          f"{(max(r[3] for r in rows) - t0) / 1e3:.1f} us from the first kernel's start to the last one's end")
    print("kernel | first block starts us | let go by the kernels before us | last block ends us | "
          "from let go to end us | from the end of the one before to this end us")
    prev_end = None
    for word, start, rel, end in rows:
        kind, extra = word % 256, word // 256
        name = TRACE_KINDS.get(kind, str(kind))
        if kind == 3:
            name += f" N={extra // 16} mode={extra % 16}"
        elif kind in (4, 5):
            name += f" splits={extra}"
        step_ = "" if prev_end is None else f"{(end - prev_end) / 1e3:.2f}"
        print(f"{name} | {(start - t0) / 1e3:.2f} | {(rel - t0) / 1e3:.2f} | {(end - t0) / 1e3:.2f} | "
              f"{(end - rel) / 1e3:.2f} | {step_}")
        prev_end = end
    # a layer's period: from the end of one q/k/v product to the end of the next
    qkv_ends = [end for word, _, _, end in rows if word % 256 == 3 and (word // 256) % 16 == 0
                and (word // 256) // 16 == (cfg["num_attention_heads"] + 2 * cfg["num_key_value_heads"]) * cfg["head_dim"]]
    if len(qkv_ends) > 2:
        periods = [(b - a) / 1e3 for a, b in zip(qkv_ends[1:-1], qkv_ends[2:])]
        print(f"layer period (end of a q/k/v product to the end of the next): "
              f"{sum(periods) / len(periods):.2f} us over {len(periods)} layers")
    eng.end_sequences(slots)


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("what", choices=["gemm", "attn-decode", "attn-prefill", "elementwise", "step", "timeline", "decode"])
    ap.add_argument("sizes", type=int, nargs="+")
    ap.add_argument("--iters", type=int, default=50)
    ap.add_argument("--layers", type=int, default=4, help="layers of the model that `step` builds")
    ap.add_argument("--model", default="mistral7b", choices=sorted(MODEL_SIZES),
                    help="step, timeline: whose layer sizes the model has")
    ap.add_argument("--window", type=int, default=0, help="decode: the sliding window (0: none)")
    ap.add_argument("--equal-shares", action="store_true",
                    help="decode: every sequence's keys in equal shares (no page quantum)")
    ap.add_argument("--splits", type=int, default=0,
                    help="attn-decode, timeline: this many key splits instead of the engine's choice")
    a = ap.parse_args()
    global SIZES
    SIZES = MODEL_SIZES[a.model]
    if a.splits:
        from .csrc import attention_bf16
        attention_bf16.decode_splits = lambda *args, **kw: a.splits
    if a.what == "gemm":
        gemm(*a.sizes[:4], a.iters)
    elif a.what == "elementwise":
        elementwise(a.sizes[0], min(a.iters, 24))
    elif a.what == "timeline":
        timeline(a.sizes[0], a.sizes[1], a.layers)
    elif a.what == "step":
        step(a.sizes[0], a.sizes[1], a.sizes[2], a.layers, min(a.iters, 8))
    elif a.what == "decode":
        decode(a.sizes, a.layers, a.window or None, a.equal_shares)
    elif a.what == "attn-decode":
        attn_decode(a.sizes[0], a.sizes[1], a.iters)
    else:
        attn_prefill(a.sizes[0], a.iters)


if __name__ == "__main__":
    main()
