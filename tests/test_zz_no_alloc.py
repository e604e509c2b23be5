"""The decode attention entry point that allocates nothing (csrc/attention_decode_noalloc.h).

Some callers of these kernels cannot call cudaMalloc: a plugin in a host program that
owns the device heap, a real-time loop that may not wait on the allocator, a process
that has handed all free memory to its own pool.  For them the library has one entry
point whose scratch is a fixed array inside the library.  This test calls it the way
such a caller would, through its exported C symbol with raw pointers, twice in a row,
and checks each result against the ordinary entry point, which takes its scratch from
the caller.  It also checks that a request beyond the fixed scratch is refused.

The file name makes pytest collect it after every other test.
"""
import ctypes
import math
from ctypes import c_float, c_int, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
HD = 128


def _args(q, pc, out, seq_len, nh, nkv, window, n_splits, scratch=None):
    a = [c_void_p(q.data_ptr()), c_void_p(pc.k_pages.data_ptr()), c_void_p(pc.v_pages.data_ptr()),
         c_void_p(out.data_ptr())]
    if scratch is not None:
        a.append(c_void_p(scratch.data_ptr()))
    a += [c_void_p(seq_len.data_ptr()), c_void_p(pc.seq_slot.data_ptr()),
          c_void_p(pc.table.data_ptr()), c_int(pc.table.stride(0)), c_int(q.shape[0]), c_int(nh),
          c_int(nkv), c_int(window), c_float(1 / math.sqrt(HD)), c_int(n_splits),
          c_void_p(torch.cuda.current_stream().cuda_stream)]
    return a


def test_no_alloc_decode_matches_ordinary_entry_point():
    from test_kernels_gpu import Paged, _rand
    from torchless_rs_b200.csrc import attention_bf16  # noqa: F401  (registers the libraries)
    from torchless_rs_b200.csrc import build

    ordinary = ctypes.CDLL(build.build_library(f"attn_bf16_hd{HD}"))
    noalloc = ctypes.CDLL(build.build_library(f"attn_noalloc_bf16_hd{HD}"))
    f_ord = getattr(ordinary, f"tl_attn_decode_hd{HD}")
    f_new = getattr(noalloc, f"tl_attn_decode_noalloc_hd{HD}")
    f_floats = getattr(ordinary, f"tl_attn_decode_scratch_floats_hd{HD}")
    f_floats.restype = ctypes.c_longlong
    f_err = noalloc.tl_attn_decode_noalloc_error
    f_err.restype = ctypes.c_char_p
    for f in (f_ord, f_new):
        f.restype = c_int

    nh, nkv = 8, 2
    # two calls in a row with different inputs, sizes and split counts: the second must
    # not be disturbed by what the first left in the shared scratch
    for call, (lens, window, n_splits, seed) in enumerate(
            [([700, 33, 129, 64], 0, 6, 1), ([90, 300], 100, 3, 2)]):
        pc = Paged(lens, nkv, HD, torch.bfloat16, 60 + seed)
        B = len(lens)
        q = _rand((B, nh * HD), torch.bfloat16, 70 + seed)
        seq_len = torch.tensor(lens, dtype=torch.int32, device=DEV)
        want = torch.empty((B, nh * HD), dtype=torch.bfloat16, device=DEV)
        scratch = torch.empty(f_floats(c_int(B), c_int(nh), c_int(n_splits)),
                              dtype=torch.float32, device=DEV)
        assert f_ord(*_args(q, pc, want, seq_len, nh, nkv, window, n_splits, scratch)) == 0
        got = torch.full_like(want, float("nan"))
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        rc = f_new(*_args(q, pc, got, seq_len, nh, nkv, window, n_splits))
        assert rc == 0, f_err(c_int(rc)).decode()
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        assert torch.isfinite(got.float()).all(), f"call {call}: output not written"
        assert torch.allclose(got.float(), want.float(), rtol=2e-2, atol=2e-2), f"call {call}"

    # beyond the fixed scratch: refused with a message, nothing launched
    B, n_splits = 64, 64      # 64 * 8 * 64 * 130 floats > 2 Mi
    pc = Paged([40] * B, nkv, HD, torch.bfloat16, 99)
    q = _rand((B, nh * HD), torch.bfloat16, 98)
    seq_len = torch.tensor([40] * B, dtype=torch.int32, device=DEV)
    out = torch.zeros((B, nh * HD), dtype=torch.bfloat16, device=DEV)
    rc = f_new(*_args(q, pc, out, seq_len, nh, nkv, 0, n_splits))
    assert rc == -3
    assert b"exceeds the fixed scratch" in f_err(c_int(rc))
    torch.cuda.synchronize()
    assert not out.any()
