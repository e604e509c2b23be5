"""bin/trace_run as a user drives it: the same requests whole, with the last 32 tokens
one by one, and in batches of unequal lengths whose shorter requests end earlier, one
batch after another in a cache that only holds one; all compared with the plain
implementation, in 32-bit and in bfloat16."""
import json
import os
import shutil
import subprocess
import tempfile

import numpy as np
import pytest

from helpers_gpu import assert_close
from plain import mistral_plain as plain
from tiny import CONFIGS, make_model_dir, random_tokens, read_weights_numpy

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run_trace(model_dir, dtype, max_tokens, steps):
    """Feeds the step records and returns {step: array [wanted, vocab]}; checks the
    protocol (one `done` line per step, files only where something was wanted)."""
    out = tempfile.mkdtemp(prefix="tl_trace_")
    p = subprocess.Popen([os.path.join(ROOT, "bin", "trace_run"), "--model", model_dir, "--dtype", dtype,
                          "--out", out, "--max-tokens", str(max_tokens)],
                         stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True)
    for rec in steps:
        p.stdin.write(json.dumps(rec) + "\n")
        p.stdin.flush()
        line = p.stdout.readline().strip()       # the next step may come only after this
        assert line == f"done {rec['step']}", line
    p.stdin.close()
    assert p.wait(timeout=300) == 0
    vocab = json.load(open(os.path.join(model_dir, "config.json")))["vocab_size"]
    got = {}
    for rec in steps:
        f = os.path.join(out, f"{rec['step']}.f32")
        n = sum(len(e.get("want", [])) for e in rec["entries"])
        assert os.path.exists(f) == (n > 0)
        if n:
            got[rec["step"]] = np.fromfile(f, dtype="<f4").reshape(n, vocab)
    shutil.rmtree(out, ignore_errors=True)
    return got


def collect(steps, got):
    """{request id: {position: logits row}} from the step records and outputs."""
    pos, out = {}, {}
    for rec in steps:
        row = 0
        for e in rec["entries"]:
            p0 = pos.get(e["id"], 0)
            for w in e.get("want", []):
                out.setdefault(e["id"], {})[p0 + w] = got[rec["step"]][row]
                row += 1
            pos[e["id"]] = p0 + len(e["tokens"])
    return out


def check(cfg, weights, reqs, steps, got, dtype):
    by_req = collect(steps, got)
    for rid, toks in reqs.items():
        ref = plain.forward_logits(cfg, weights, toks)
        rows = by_req[rid]
        assert sorted(rows) == list(range(len(toks))), f"{rid}: positions {sorted(rows)[:5]}..."
        assert_close(np.stack([rows[i] for i in range(len(toks))]), ref, dtype, f"request {rid}")


@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("A", "bfloat16"), ("D", "float32"),
                                        ("D", "bfloat16"), ("C", "bfloat16")])
def test_three_ways_of_cutting(name, dtype):
    cfg = CONFIGS[name]
    d = make_model_dir(cfg, 41)
    w = read_weights_numpy(d)
    rng = np.random.default_rng(8)
    lens = {"a": 70, "b": 33, "c": 120, "d": 45, "e": 64}
    reqs = {k: random_tokens(rng, n, cfg["vocab_size"]) for k, n in lens.items()}
    all_ = lambda n: list(range(n))
    # 1. each request alone and whole
    steps = [{"step": i, "entries": [{"id": k, "tokens": t, "want": all_(len(t))}], "end": [k]}
             for i, (k, t) in enumerate(reqs.items())]
    check(cfg, w, reqs, steps, run_trace(d, dtype, 128, steps), dtype)
    # 2. the last 32 tokens one by one
    steps, n = [], 0
    for k, t in reqs.items():
        head = len(t) - 32
        steps.append({"step": n, "entries": [{"id": k, "tokens": t[:head], "want": all_(head)}], "end": []})
        n += 1
        for i in range(head, len(t)):
            steps.append({"step": n, "entries": [{"id": k, "tokens": [t[i]], "want": [0]}],
                          "end": [k] if i == len(t) - 1 else []})
            n += 1
    check(cfg, w, reqs, steps, run_trace(d, dtype, 128, steps), dtype)
    # 3. batches of unequal lengths; shorter requests end earlier; the cache holds one batch
    steps, n = [], 0
    for batch, prefix in ((["a", "b", "c"], {"a": 20, "b": 31, "c": 3}), (["d", "e"], {"d": 44, "e": 1})):
        fed = dict(prefix)
        live = list(batch)
        ends = [k for k in live if fed[k] == len(reqs[k])]
        steps.append({"step": n, "entries": [{"id": k, "tokens": reqs[k][:fed[k]], "want": all_(fed[k])}
                                             for k in live], "end": ends})
        n += 1
        live = [k for k in live if k not in ends]
        while live:
            entries = [{"id": k, "tokens": [reqs[k][fed[k]]], "want": [0]} for k in live]
            for k in live:
                fed[k] += 1
            ends = [k for k in live if fed[k] == len(reqs[k])]
            steps.append({"step": n, "entries": entries, "end": ends})
            n += 1
            live = [k for k in live if k not in ends]
    need = max(sum((lens[k] + 63) // 64 * 64 for k in b) for b in (["a", "b", "c"], ["d", "e"]))
    check(cfg, w, reqs, steps, run_trace(d, dtype, need, steps), dtype)


def test_steps_without_wanted_logits_write_no_file():
    cfg = CONFIGS["B"]
    d = make_model_dir(cfg, 42)
    w = read_weights_numpy(d)
    toks = random_tokens(np.random.default_rng(9), 10, cfg["vocab_size"])
    steps = [{"step": 0, "entries": [{"id": "x", "tokens": toks[:6], "want": []}], "end": []},
             {"step": 1, "entries": [{"id": "x", "tokens": toks[6:], "want": [3]}], "end": ["x"]}]
    got = run_trace(d, "float32", 64, steps)
    assert list(got) == [1]
    assert_close(got[1], plain.forward_logits(cfg, w, toks)[9:10], "float32", "last position")
