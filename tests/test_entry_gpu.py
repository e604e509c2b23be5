"""Generation through the Python entry point and the command line, the replay
program as a user runs it, and the sampling kernels."""
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from helpers_gpu import TinyModel
from plain import mistral_plain as plain
from tiny import CONFIGS, make_model_dir, random_tokens, read_weights_numpy

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _plain_greedy(tm, prompt, n, stop=()):
    seq, out = list(prompt), []
    for _ in range(n):
        t = int(np.argmax(tm.reference(seq)[-1]))
        if t in stop:
            break
        out.append(t)
        seq.append(t)
    return out


@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("B", "float32"), ("D", "float32")])
def test_greedy_generation_equals_plain(name, dtype):
    tm = TinyModel(name, dtype, seed=21, max_tokens=512)
    rng = np.random.default_rng(4)
    lens = [5, 11, 23] if name == "A" else [1, 19, 40]
    prompts = [random_tokens(rng, n, tm.cfg["vocab_size"]) for n in lens]
    res = tm.model.generate(prompts, max_tokens=12, temperature=0.0, stop_ids=())
    for p, r in zip(prompts, res):
        assert r.tokens == _plain_greedy(tm, p, 12), f"prompt of {len(p)}"
        assert not r.stopped_at_eos and r.prompt_len == len(p)
    # a stop token ends its sequence early and is not emitted; the others go on
    first = res[1].tokens
    stop = first[3]
    regrouped, copied = tm.engine.steps_regrouped_on_device, tm.engine.stager.bytes_copied
    res2 = tm.model.generate(prompts, max_tokens=12, temperature=0.0, stop_ids=[stop])
    want = _plain_greedy(tm, prompts[1], 12, stop=(stop,))
    assert res2[1].tokens == want and res2[1].stopped_at_eos
    for i in (0, 2):
        assert res2[i].tokens == _plain_greedy(tm, prompts[i], 12, stop=(stop,)), f"prompt {i} beside the one that ended"
    # the batch shrank on the way: the steps after that were set up by a kernel, and the host laid
    # out the prompts' step and the first decode step only
    if not all(r.stopped_at_eos for r in res2) and len(want) < 10:
        assert tm.engine.steps_regrouped_on_device > regrouped
        T, B = sum(len(p) for p in prompts), len(prompts)
        pad = lambda n: (n + 3) // 4 * 4
        layout = lambda t: 4 * (4 * pad(t) + 3 * pad(B) + pad(B + 1))     # bytes of one step's eight arrays
        assert tm.engine.stager.bytes_copied - copied == layout(T) + layout(B)
    assert tm.engine.cache.slots.held_count == 0
    tm.engine.cache.check()


def test_generation_in_bfloat16_follows_plain_where_the_margin_allows():
    tm = TinyModel("D", "bfloat16", seed=22, max_tokens=512)
    rng = np.random.default_rng(5)
    prompts = [random_tokens(rng, n, tm.cfg["vocab_size"]) for n in (3, 30, 70)]
    res = tm.model.generate(prompts, max_tokens=10, temperature=0.0, stop_ids=())
    for p, r in zip(prompts, res):
        seq = list(p)
        for tok in r.tokens:
            logits = tm.reference(seq)[-1]
            best = int(np.argmax(logits))
            if tok != best:   # only where the two best plain logits are within the bfloat16 tolerance
                assert logits[best] - logits[tok] < 2.5e-2 * np.abs(logits).max()
            seq.append(tok)


def test_many_requests_run_batch_after_batch():
    tm = TinyModel("B", "float32", seed=23, max_tokens=256, max_batch=3)
    rng = np.random.default_rng(6)
    prompts = [random_tokens(rng, int(n), tm.cfg["vocab_size"]) for n in rng.integers(1, 40, 8)]
    res = tm.model.generate(prompts, max_tokens=5, temperature=0.0, stop_ids=())
    for p, r in zip(prompts, res):
        assert r.tokens == _plain_greedy(tm, p, 5)
    assert tm.engine.cache.slots.held_count == 0


def test_temperature_sampling_equals_plain_draws():
    from torchless_rs_b200.sampling.params import uniform_for
    tm = TinyModel("B", "float32", seed=24, max_tokens=512)
    rng = np.random.default_rng(7)
    prompts = [random_tokens(rng, n, tm.cfg["vocab_size"]) for n in (1, 19)]
    for kw in (dict(temperature=0.8), dict(temperature=1.3, top_k=20), dict(temperature=0.9, top_p=0.7)):
        res = tm.model.generate(prompts, max_tokens=12, stop_ids=(), seed=11, **kw)
        for i, (p, r) in enumerate(zip(prompts, res)):
            seq = list(p)
            for k, tok in enumerate(r.tokens):
                probs = plain.sample_probs(tm.reference(seq)[-1], kw["temperature"], kw.get("top_k"),
                                           kw.get("top_p"))
                u = uniform_for(11, i, k)
                c = np.cumsum(probs)
                want = plain.draw(probs, u)
                if tok != want:   # the draw may differ only if u falls within rounding of a boundary
                    assert np.min(np.abs(c - u)) < 1e-5, f"{kw} request {i} token {k}"
                seq.append(tok)


@pytest.mark.parametrize("V", [331, 32000])
def test_sampling_kernels_alone(V):
    from torchless_rs_b200.sampling.params import SamplingParams
    from torchless_rs_b200.sampling.sampler import Sampler
    s = Sampler("cuda:0")
    g = torch.Generator().manual_seed(V)
    logits = (torch.randn((6, V), generator=g) * 3).cuda()
    logits[2, 5] = logits[2, 77] = logits[2].max() + 1      # a tie: the highest index wins, as in the reference
    assert s.select(logits, SamplingParams.greedy()).tolist() == [plain.greedy(row) for row in logits.cpu().numpy()]
    assert plain.greedy(logits[2].cpu().numpy()) == 77
    many = (torch.randn((70, V), generator=g) * 3).cuda()      # 64 rows and more: one block per row
    many[3, 5] = many[3, 77] = many[3].max() + 1
    assert s.select(many, SamplingParams.greedy()).tolist() == [plain.greedy(row) for row in many.cpu().numpy()]
    ln = logits.cpu().numpy()
    for kw in (dict(temperature=0.7), dict(temperature=1.0, top_k=5), dict(temperature=1.0, top_k=1),
               dict(temperature=1.5, top_p=0.3), dict(temperature=0.9, top_k=50, top_p=0.9),
               dict(temperature=1.0, top_k=V + 5, top_p=1.0)):
        us = [0.0, 0.13, 0.5, 0.77, 0.999, 0.31]
        got = s.select(logits, SamplingParams(**kw), us).tolist()
        for r in range(6):
            probs = plain.sample_probs(ln[r], kw["temperature"], kw.get("top_k"), kw.get("top_p"))
            assert probs[got[r]] > 0, f"{kw} row {r}: token outside the kept set"
            want = plain.draw(probs, us[r])
            if got[r] != want:
                assert np.min(np.abs(np.cumsum(probs) - us[r])) < 1e-5, f"{kw} row {r}"
    # hotter is flatter, colder is sharper (reference: sampler/tests.rs:92-134): count distinct draws
    us = [i / 64 + 0.003 for i in range(6)]
    row = logits[:1].expand(6, V).contiguous()
    cold = len(set(s.select(row, SamplingParams(temperature=0.05), us).tolist()))
    hot = len(set(s.select(row, SamplingParams(temperature=5.0), us).tolist()))
    assert cold <= hot


def test_command_line_ids_in_ids_out():
    d = make_model_dir(CONFIGS["A"], 31)
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "torchless"), "--temperature", "0",
                        "--max-tokens", "6", "--dtype", "float32", d, "3 17 200 ; 45, 9"],
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr
    lines = [l.split() for l in r.stdout.strip().splitlines()]
    assert len(lines) == 2 and all(len(l) == 6 for l in lines)
    w = read_weights_numpy(d)
    for prompt, line in zip(([3, 17, 200], [45, 9]), lines):
        seq = list(prompt)
        for tok in line:
            assert int(tok) == int(np.argmax(plain.forward_logits(CONFIGS["A"], w, seq)[-1]))
            seq.append(int(tok))
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "torchless"), "--bogus", d],
                       capture_output=True, text=True, timeout=120)
    assert r.returncode == 1 and "unknown option" in r.stderr


def test_command_line_random_weights(tmp_path):
    """--random-weights needs config.json only; --save-weights writes the folder's tensors, and
    a second run that reads them gives the same tokens."""
    import json
    import torchless_rs_b200 as tl
    d = str(tmp_path)
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(tl.config_from_dict(CONFIGS["B"]).to_dict(), f)
    common = ["--temperature", "0", "--max-tokens", "5", "--dtype", "float32"]
    exe = [sys.executable, os.path.join(ROOT, "bin", "torchless")]
    r1 = subprocess.run(exe + common + ["--random-weights", "--weights-seed", "4", "--save-weights", d, "7 8 9"],
                        capture_output=True, text=True, timeout=600)
    assert r1.returncode == 0, r1.stderr
    assert os.path.isfile(os.path.join(d, "model.safetensors"))
    r2 = subprocess.run(exe + common + [d, "7 8 9"], capture_output=True, text=True, timeout=600)
    assert r2.returncode == 0, r2.stderr
    assert r1.stdout.split() == r2.stdout.split() and len(r1.stdout.split()) == 5
    w = read_weights_numpy(d)
    seq = [7, 8, 9]
    for tok in r1.stdout.split():
        assert int(tok) == int(np.argmax(plain.forward_logits(CONFIGS["B"], w, seq)[-1]))
        seq.append(int(tok))


def test_model_drawn_on_the_device_is_the_folder_written_from_the_same_seed(tmp_path):
    """`from_random` draws weights on the device; `write_random_model` on the host writes the
    same values from the same seed, so the plain implementation can follow a model that never
    was a folder."""
    import numpy as np
    import torchless_rs_b200 as tl
    from plain import mistral_plain as plain
    from tiny import TINY_B, read_weights_numpy
    cfg = tl.config_from_dict(TINY_B)
    m = tl.from_random(cfg, seed=21, dtype="float32", max_tokens=256)
    d = tl.write_random_model(cfg, str(tmp_path), 21, torch.float32, "cpu")
    w = read_weights_numpy(d)
    toks = [int(t) for t in np.random.default_rng(1).integers(0, TINY_B["vocab_size"], 25)]
    (s,) = m.start_sequences(1)
    got = m.step([s], [toks], "all").cpu().numpy()
    m.end_sequences([s])
    ref = plain.forward_logits(TINY_B, w, toks)
    assert (np.abs(got - ref) <= 5e-5 + 1e-4 * np.abs(ref)).all()
    m2 = tl.load(d, dtype="float32", max_tokens=256)
    (s,) = m2.start_sequences(1)
    assert np.array_equal(m2.step([s], [toks], "all").cpu().numpy(), got)
    # and `load(..., random_weights=True)` needs config.json only
    import os
    os.remove(os.path.join(d, "model.safetensors"))
    m3 = tl.load(d, dtype="float32", max_tokens=256, random_weights=True, seed=21)
    (s,) = m3.start_sequences(1)
    assert np.array_equal(m3.step([s], [toks], "all").cpu().numpy(), got)
