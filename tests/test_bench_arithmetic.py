"""The byte and flop counts that bench.py divides by, against the numbers worked out by hand
for the sizes of Mistral 7B (parameter count after the reference's src/loader/gpu_memory.rs:693-724,
cache bytes per token after :734-746), and its behaviour for more than one GPU."""
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import bench  # noqa: E402


def test_decode_bytes_and_prefill_flops_of_mistral_7b():
    cfg = bench.MISTRAL_7B
    # per layer: q/k/v 6144 x 4096, o 4096 x 4096, gate, up and down 3 x 14336 x 4096, two norm weights
    per_layer = 6144 * 4096 + 4096 * 4096 + 3 * 14336 * 4096 + 2 * 4096
    assert bench.weight_bytes_per_step(cfg, 32) == 2 * (32 * per_layer + 32000 * 4096 + 4096)
    assert abs(bench.weight_bytes_per_step(cfg, 32) / 1e9 - 14.22) < 0.01
    # keys and values of 8 heads of 128 in 32 layers, 2 bytes each
    assert bench.kv_bytes_per_token(cfg, 32) == 131072
    # 2 flops per weight and token, the causal half of attention, and the head for one row
    assert abs(bench.prefill_flops(cfg, 32, 2048) / 1e12 - 29.69) < 0.01
    assert bench.weight_bytes_per_step(cfg, 4) < bench.weight_bytes_per_step(cfg, 32) / 7


def test_more_than_one_gpu_is_refused_with_exit_code_2():
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--gpus", "2"],
                       capture_output=True, text=True, timeout=120)
    assert r.returncode == 2
    assert len(r.stdout.strip().splitlines()) == 1 and "one GPU" in r.stdout


def test_reference_arm_says_why_it_is_unavailable():
    import json
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference"],
                       capture_output=True, text=True, timeout=120)
    assert r.returncode == 0
    rec = json.loads(r.stdout.strip().splitlines()[-1])
    assert rec["impl"] == "reference" and rec["unavailable"]
