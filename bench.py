"""Measurement of decode and prefill throughput at Mistral-family sizes on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]
                    [--config mistral7b|nemo12b|small22b]

Prints one JSON line.  A "step" is one decode step of the whole batch.  The default
run: random weights of the sizes of Mistral-7B-v0.1, batch 8, every sequence ending
at a context of 4096 tokens.  The other two configurations (Mistral-NeMo-12B sizes with 8
prompts of 8192 tokens; Mistral-Small-22B sizes with 16 prompts of 128 to 4096 tokens and 256
decoded tokens each) print a record of the same shape.  `value` is decoded tokens per second timed on the device
(CUDA events around K steps of step + token selection); `e2e` is the same through the
Python entry point `Model.generate`, host token ids in and out each step, timed by
the host between the first and the last emitted token.  Inputs exceed the L2 cache
(14 GB of weights are read each step), so no flush is needed between steps.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

_ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, _ROOT)

# the sizes of Mistral-7B-v0.1 (the benchmark's third configuration)
MISTRAL_7B = dict(
    architectures=["MistralForCausalLM"], model_type="mistral", num_hidden_layers=32,
    hidden_size=4096, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
    intermediate_size=14336, vocab_size=32000, rope_theta=10000.0, sliding_window=4096,
    rms_norm_eps=1e-5, max_position_embeddings=32768, tie_word_embeddings=False)
NEMO_12B = dict(MISTRAL_7B, num_hidden_layers=40, hidden_size=5120, vocab_size=131072,
                rope_theta=1000000.0, sliding_window=None, max_position_embeddings=131072)
SMALL_22B = dict(MISTRAL_7B, num_hidden_layers=56, hidden_size=6144, num_attention_heads=48,
                 intermediate_size=16384, vocab_size=32768, rope_theta=1000000.0, sliding_window=None)
CONTEXT = 4096
PREFILL_TOKENS = 2048


def small22b_lengths():
    """16 prompt lengths, uniform in 128..4096, from a fixed seed."""
    import random
    r = random.Random(22)
    return [r.randint(128, 4096) for _ in range(16)]


# name -> (config.json keys, model name, prompt lengths of the end-to-end run, decoded tokens there)
WORKLOADS = {
    "mistral7b": (MISTRAL_7B, "Mistral-7B-v0.1 sizes", None, None),
    "nemo12b": (NEMO_12B, "Mistral-NeMo-12B sizes", [8192] * 8, 64),
    "small22b": (SMALL_22B, "Mistral-Small-22B sizes", small22b_lengths(), 256),
}
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def load_peaks() -> dict:
    p = os.path.join(_ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(p):
        with open(p) as f:
            d = json.load(f)
        d["source"] = "measured"
        return d
    return dict(FALLBACK_PEAKS)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), [c.strip() for c in line.split(",")]))

    def mark(self):
        return time.time()

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()

    def summary(self, t0: float, t1: float) -> dict:
        rows = [r for t, r in self.rows if t0 <= t <= t1 and len(r) >= 6] or \
               [r for _, r in self.rows if len(r) >= 6]
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        mhz = [float(r[0]) for r in rows if r[0].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[2 + i].lower() == "active" for r in rows)]
        return {"sm_mhz": statistics.median(mhz) if mhz else None,
                "sm_max_mhz": float(rows[0][1]) if rows[0][1].replace(".", "").isdigit() else None,
                "reasons": reasons, "samples": len(rows)}


def weight_bytes_per_step(cfg: dict, n_layers: int, elt: int = 2) -> int:
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    nh, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    per_layer = ((nh + 2 * nkv) * hd * H + nh * hd * H + 3 * I * H + 2 * H) * elt
    return n_layers * per_layer + (V * H + H) * elt


def kv_bytes_per_token(cfg: dict, n_layers: int, elt: int = 2) -> int:
    return 2 * n_layers * cfg["num_key_value_heads"] * cfg["head_dim"] * elt


def prefill_flops(cfg: dict, n_layers: int, n) -> float:
    """`n`: the tokens of one prompt, or the list of the lengths of a batch of prompts."""
    lens = [n] if isinstance(n, int) else list(n)
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    nh, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    per_layer = (nh + 2 * nkv) * hd * H + nh * hd * H + 3 * I * H
    w = cfg.get("sliding_window")
    # causal attention: each query sees min(position + 1, window) keys; 4 flops per key and dimension
    seen = sum(sum(min(p + 1, w) if w else p + 1 for p in range(L)) for L in lens) if w else \
        sum(L * (L + 1) // 2 for L in lens)
    return (2.0 * sum(lens) * per_layer * n_layers + 4.0 * nh * hd * seen * n_layers
            + 2.0 * V * H * len(lens))


def fill_context(model, batch: int, context):
    """Takes `batch` slots and gives each a context of `context` tokens (a number, or one per
    slot) of synthetic cache content (random keys and values), without running a prefill."""
    import torch
    eng = model.engine
    slots = eng.start_sequences(batch)
    lens = [context] * batch if isinstance(context, int) else list(context)
    eng.cache.prepare(slots, lens)
    eng.cache.commit(slots, lens)
    return slots


def decode_device_timed(model, batch: int, steps: int, warmup: int, end_context):
    """K decode steps (step + greedy selection) timed with CUDA events; the sequences
    end at `end_context` tokens (a number, or one per sequence).  Returns (tokens/s, ms per
    step, mean context, launches in the timed region)."""
    import torch
    from torchless_rs_b200.csrc import ops
    from torchless_rs_b200.sampling.params import SamplingParams
    eng = model.engine
    ends = [end_context] * batch if isinstance(end_context, int) else list(end_context)
    slots = fill_context(model, batch, [e - steps - warmup for e in ends])
    toks = [[(7 * i + 3) % eng.vocab_size] for i in range(batch)]
    greedy = SamplingParams.greedy()
    for _ in range(warmup):
        model.sampler.select(eng.step(slots, toks, "last"), greedy)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    l0 = ops.launches()
    e0.record()
    for _ in range(steps):
        model.sampler.select(eng.step(slots, toks, "last"), greedy)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    launches = ops.launches() - l0
    eng.end_sequences(slots)
    mean_ctx = sum(ends) / batch - steps / 2.0
    return batch / (ms / 1e3), ms, mean_ctx, launches


def decode_end_to_end(model, batch: int, steps: int, warmup: int, end_context: int):
    """The same through `Model.generate`: host token ids in, host token ids out at every
    step.  Real prompts are prefilled first (not timed); the time runs on the host from
    the token emitted after `warmup` decode steps to the last one; a stamp is taken when the
    host holds the step's tokens."""
    import torch
    eng = model.engine
    # the clocks sag for some twenty steps after the 32k-token prefill of the prompts (power
    # cap); those steps are warm-up here, so that both numbers are taken at steady clocks
    warmup = max(warmup, 24)
    n_prompt = end_context - steps - warmup - 1
    prompts = [[(11 * i + 5 * j + 3) % eng.vocab_size for j in range(n_prompt)] for i in range(batch)]
    stamps = []

    def on_token(i, tok):
        if i == batch - 1:    # the host holds this step's tokens now (they were read from the device)
            stamps.append((time.perf_counter(), eng.h2d_bytes(),
                           model._reader.bytes_copied if model._reader is not None else 0))
    advanced = eng.steps_advanced_on_device
    model.generate(prompts, max_tokens=steps + warmup + 1, temperature=0.0, stop_ids=(),
                   on_token=on_token)
    dt = stamps[-1][0] - stamps[warmup][0]
    n = len(stamps) - 1 - warmup
    # bytes counted where they are copied: step layouts and page-table rows in, selected tokens out
    h2d = (stamps[-1][1] - stamps[warmup][1]) / n
    d2h = (stamps[-1][2] - stamps[warmup][2]) / n
    return batch * n / dt, 1e3 * dt / n, h2d, d2h, eng.steps_advanced_on_device - advanced


def prefill_timed(model, lengths, repeats: int = 3):
    """One prefill step of prompts of the given lengths (a number = one prompt), timed with CUDA
    events; the median of `repeats` runs after one that is not counted."""
    import torch
    eng = model.engine
    lens = [lengths] if isinstance(lengths, int) else list(lengths)
    toks = [[(13 * i + 7 * b + 1) % eng.vocab_size for i in range(n)] for b, n in enumerate(lens)]
    times = []
    for r in range(repeats + 1):
        slots = eng.start_sequences(len(lens))
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        eng.prefill(slots, toks)   # what `generate` calls: many tokens go in several steps
        e1.record()
        torch.cuda.synchronize()
        eng.end_sequences(slots)
        if r > 0:
            times.append(e0.elapsed_time(e1))
    return statistics.median(times), times


def generate_timed(model, lengths, new_tokens: int):
    """The workload of a configuration through `Model.generate`: prompts of the given lengths,
    `new_tokens` decoded tokens each.  Returns (ms until the host holds every first token, ms
    per decode step after that)."""
    eng = model.engine
    prompts = [[(11 * i + 5 * j + 3) % eng.vocab_size for j in range(n)] for i, n in enumerate(lengths)]
    last = len(prompts) - 1
    stamps = []
    t0 = time.perf_counter()
    model.generate(prompts, max_tokens=new_tokens, temperature=0.0, stop_ids=(),
                   on_token=lambda i, tok: stamps.append(time.perf_counter()) if i == last else None)
    return 1e3 * (stamps[0] - t0), 1e3 * (stamps[-1] - stamps[0]) / max(1, len(stamps) - 1)


def cpu_baseline(cfg: dict, n_layers: int, context: int) -> dict:
    """Times the plain C++ restatement under tests/plain (the reference's own shape of the
    computation: one token of one sequence per pass, sequential 32-bit dot products, one CPU
    thread) on one layer and the head at these layer sizes, and extends it to all layers.  The
    reference itself cannot be built where this runs (a Rust crate, no Rust toolchain)."""
    import shutil
    import tempfile
    src = os.path.join(_ROOT, "tests", "plain", "mistral_plain_onetoken.cpp")
    cxx = shutil.which("g++") or shutil.which("c++")
    if cxx is None or not os.path.isfile(src):
        return {"unavailable": "no C++ compiler or no tests/plain source"}
    with tempfile.TemporaryDirectory() as d:
        exe, cj = os.path.join(d, "plain"), os.path.join(d, "config.json")
        try:
            subprocess.run([cxx, "-O2", "-std=c++17", "-o", exe, src], check=True, capture_output=True)
            with open(cj, "w") as f:
                json.dump(cfg, f)
            out = subprocess.run([exe, "--time-layer", cj, str(context), "2"], check=True,
                                 capture_output=True, text=True, timeout=600).stdout
            t = json.loads(out)
        except (subprocess.SubprocessError, OSError, ValueError) as e:
            return {"unavailable": f"the plain C++ baseline did not run: {type(e).__name__}"}
    s_per_token = n_layers * t["layer_s"] + t["head_s"]
    return {"value": round(1.0 / s_per_token, 4), "unit": "tokens/s", "batch": 1, "context": context,
            "layer_ms": round(1e3 * t["layer_s"], 2), "head_ms": round(1e3 * t["head_s"], 2),
            "what": "plain C++ restatement (tests/plain/mistral_plain_onetoken.cpp), one CPU thread, "
                    "32-bit, one layer and the head timed and extended to all layers"}


def reference_arm(args) -> int:
    print(json.dumps({
        "impl": "reference",
        "unavailable": "rglonek/torchless-rs is a Rust crate (Cargo.toml, no Python package "
                       "metadata); pip cannot install it offline and no cargo/rustc exists here"}))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=None,
                    help="fewer layers than the configuration has (named in the record)")
    ap.add_argument("--batch", type=int, default=None)
    ap.add_argument("--config", default="mistral7b", choices=sorted(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true",
                    help="skip the timed plain C++ baseline (vs_baseline is then null)")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args)
    if args.gpus != 1:
        print(f"bench.py: this library runs on one GPU; --gpus {args.gpus} is not measured")
        return 2
    args.warmup = max(args.warmup, 3)

    import torch
    import torchless_rs_b200 as tl
    from torchless_rs_b200.config import config_from_dict

    peaks = load_peaks()
    base_cfg, model_name, prompt_lens, new_tokens = WORKLOADS[args.config]
    cfg = dict(base_cfg)
    full_layers = cfg["num_hidden_layers"]
    n_layers = args.layers or full_layers
    cfg["num_hidden_layers"] = n_layers
    config = config_from_dict(cfg)
    default = args.config == "mistral7b"
    B = args.batch or (8 if default else len(prompt_lens))
    # the contexts at which the decode steps end, and what the prefill measurement runs
    if default:
        ends, context, prefill_lens = CONTEXT, CONTEXT, PREFILL_TOKENS
        big = max(B, 64)
        cache_tokens = big * CONTEXT
    else:
        ends = [n + new_tokens for n in prompt_lens[:B]]
        context = max(ends)
        prefill_lens = prompt_lens[:B]
        big = B
        cache_tokens = sum((e + 63) // 64 * 64 for e in ends)
    model = tl.from_random(config, seed=0, dtype="bfloat16", max_tokens=cache_tokens,
                           max_batch=big, max_seq_len=(context + 63) // 64 * 64)
    for g in model.engine.cache.paged:   # synthetic cache content
        g.storage.normal_(0.0, 0.5)
    wbytes = weight_bytes_per_step(cfg, n_layers)
    kvb = kv_bytes_per_token(cfg, n_layers)

    clocks = ClockSampler()
    clocks.start()
    time.sleep(0.3)
    t0 = clocks.mark()
    tps, ms, mean_ctx, launches = decode_device_timed(model, B, args.steps, args.warmup, ends)
    t1 = clocks.mark()
    points = {}
    if default:
        e2e_tps, e2e_ms, e2e_h2d, e2e_d2h, e2e_adv = decode_end_to_end(model, B, args.steps, args.warmup, CONTEXT)
        for b, k in ((1, min(args.steps, 32)), (64, min(args.steps, 16))):
            p_tps, p_ms, _, _ = decode_device_timed(model, b, k, 3, CONTEXT)
            points[f"decode_b{b}"] = round(p_tps, 1)
            points[f"decode_b{b}_ms"] = round(p_ms, 3)
        pre_ms, pre_all = prefill_timed(model, prefill_lens, repeats=7)
    else:
        first_ms, e2e_ms = generate_timed(model, prefill_lens, new_tokens)
        e2e_tps = B / (e2e_ms / 1e3)
        e2e_h2d = e2e_d2h = e2e_adv = None
        points["first_token_ms"] = round(first_ms, 2)
        pre_ms, pre_all = prefill_timed(model, prefill_lens, repeats=3)
    clocks.stop()
    base = {"unavailable": "skipped"} if args.no_cpu_baseline else cpu_baseline(cfg, n_layers, context)

    step_bytes = wbytes + B * mean_ctx * kvb
    achieved = step_bytes / (ms / 1e3) / 1e9
    flops = prefill_flops(cfg, n_layers, prefill_lens)
    pre_tokens = prefill_lens if isinstance(prefill_lens, int) else sum(prefill_lens)
    rec = {
        "metric": f"decode tok/s ({model_name}, bf16, batch {B}, context {context})",
        "value": round(tps, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(ms, 4), "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": round(tps / base["value"], 1) if "value" in base else None,
        "baseline": base, "dtype": "bf16",
        "data": "synthetic: random weights N(0,0.02), random cache content, fixed token ids",
        "impl": "ours",
        "config": {
            "model": model_name, "layers": n_layers, "layers_of_config": full_layers,
            "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"],
            "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
            "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"],
            "sliding_window": cfg["sliding_window"], "rope_theta": cfg["rope_theta"],
            "rms_norm_eps": cfg["rms_norm_eps"],
            "global_batch": B, "seq_len": context, "mean_context": mean_ctx,
            "prefill_tokens": pre_tokens, "parallelism": "single GPU",
            "l2": "inputs_exceed_l2", "peaks": peaks["source"],
        },
        "e2e": {"value": round(e2e_tps, 1), "unit": "tokens/s", "ms_per_step": round(e2e_ms, 4),
                # measured over the timed steps where the copies are made (the default run); a step
                # of an unchanged batch copies no layout in, only page-table rows that gained a page
                "h2d_bytes_per_step": (round(e2e_h2d, 1) if e2e_h2d is not None
                                       else 4 * (8 * ((B + 3) // 4 * 4))),
                "d2h_bytes_per_step": round(e2e_d2h, 1) if e2e_d2h is not None else 4 * B,
                "steps_advanced_on_device": e2e_adv},
        "gpu_launches": launches,
        "prefill": {"value": round(pre_tokens / (pre_ms / 1e3), 1), "tokens": pre_tokens,
                    "ms": round(pre_ms, 3), "of": "median", "ms_each": [round(t, 2) for t in pre_all],
                    "frac": round(flops / (pre_ms / 1e3) / (peaks["bf16_tflops"] * 1e12), 4),
                    "peak_tflops": peaks["bf16_tflops"],
                    "frac_of_sustained": (round(flops / (pre_ms / 1e3) / (peaks["bf16_tflops_sustained"] * 1e12), 4)
                                          if peaks.get("bf16_tflops_sustained") else None)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"],
                     "unit": "GB/s", "frac": round(achieved / peaks["hbm_gbs"], 4)},
        "points": points,
        "clocks": clocks.summary(t0, t1),
    }
    print(json.dumps(rec))
    return 0


if __name__ == "__main__":
    sys.exit(main())
