"""The give-up path of the kernels' bounded waits, made to happen without a fault: a kernel
defined under tests/kernels waits, through the package's own wait helper, on a barrier at which
nobody arrives.  The wait runs out after 2^10 polls, the kernel reports and returns, and the
next ordinary launch works."""
import ctypes
import os
import subprocess
import tempfile

import pytest
import torch

pytestmark = pytest.mark.gpu

_HERE = os.path.dirname(os.path.abspath(__file__))


def _build():
    from torchless_rs_b200.csrc import build
    out = os.path.join(tempfile.mkdtemp(prefix="tl_wait_"), "libwait_runs_out.so")
    cmd = [build.find_nvcc(), *build.ARCH_FLAGS, "-O3", "-std=c++17", "-Xcompiler", "-fPIC", "-shared",
           "-I", os.path.dirname(build.__file__), "-o", out, os.path.join(_HERE, "kernels", "wait_runs_out.cu"),
           "-lcudart"]
    subprocess.run(cmd, check=True, capture_output=True)
    return ctypes.CDLL(out)


def test_a_wait_that_runs_out_reports_and_returns():
    from torchless_rs_b200.csrc.gemm_bf16 import GemmBf16
    torch.zeros(1, device="cuda:0")            # a context
    lib = _build()
    lib.test_wait_runs_out.restype = ctypes.c_int
    report = (ctypes.c_int * 3)()
    word = lib.test_wait_runs_out(report)
    assert word == 7, f"error word {word}"                   # the code of the wait that ran out
    assert list(report) == [0, 0, 7]                         # both waits returned false; the second saw the flag
    assert lib.test_wait_runs_out(report) == 7               # the word was cleared and is set again
    # the context is intact: an ordinary product of the package runs and is right
    g = GemmBf16.get()
    gen = torch.Generator().manual_seed(1)
    a = torch.randn((8, 512), generator=gen).to(torch.bfloat16).cuda()
    w = (torch.randn((256, 512), generator=gen) / 22).to(torch.bfloat16).cuda()
    out = torch.empty((8, 256), dtype=torch.float32, device="cuda:0")
    assert g.run(a, w, out, 0)
    assert torch.allclose(out.double(), a.double() @ w.double().T, rtol=1e-3, atol=1e-3)
    assert g.take_error() == 0
