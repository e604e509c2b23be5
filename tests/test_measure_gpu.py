"""The single-kernel measurement commands that the profile notes quote still run."""
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("args", [
    ["gemm", "8", "512", "1024", "0", "--iters", "3"],
    ["gemm", "8", "512", "1024", "2", "--iters", "3"],
    ["gemm", "300", "512", "1024", "1", "--iters", "3"],
    ["attn-decode", "2", "300", "--iters", "3"],
    ["attn-prefill", "256", "--iters", "2"],
    ["elementwise", "64"],
    ["decode", "700", "90", "90", "--layers", "1"],
])
def test_measure_command_runs(args):
    p = subprocess.run([sys.executable, "-m", "torchless_rs_b200.measure", *args], capture_output=True, text=True,
                       timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert " us" in p.stdout, p.stdout[-500:]
    if args[0] in ("gemm", "attn-prefill"):
        assert "error word 0" in p.stdout, p.stdout[-500:]
