"""The decode attention entry point that allocates nothing (csrc/attention_decode_noalloc.h).

Some callers of these kernels cannot call cudaMalloc: a plugin in a host program that
owns the device heap, a real-time loop that may not wait on the allocator, a process
that has handed all free memory to its own pool.  For them the library has one entry
point whose scratch is a fixed array inside the library.  This test calls it the way
such a caller would, through its exported C symbol with raw pointers, twice in a row,
and checks each result against the ordinary entry point, which takes its scratch from
the caller (the same bits are expected), and against a plain attention.  It checks that
the driver's count of free device memory does not move over the calls, and that a request
beyond the fixed scratch is refused.

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
    from test_kernels_gpu import Paged, _rand, attention_reference
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
    scale = 1 / math.sqrt(HD)
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
        if call == 0:
            # the first call on a device loads the library's module (its fixed array takes its
            # 8 MiB then) and looks up the array's address: not part of what is measured below
            rc = f_new(*_args(q, pc, got, seq_len, nh, nkv, window, n_splits))
            assert rc == 0, f_err(c_int(rc)).decode()
            got.fill_(float("nan"))
        torch.cuda.synchronize()
        # free device memory as the driver counts it: a cudaMalloc inside the library would
        # lower it, whoever's allocator made the call (torch's own counters would not see it)
        free_before = torch.cuda.mem_get_info()[0]
        for _ in range(4):
            rc = f_new(*_args(q, pc, got, seq_len, nh, nkv, window, n_splits))
            assert rc == 0, f_err(c_int(rc)).decode()
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info()[0] == free_before, "device memory was taken during the calls"
        assert torch.isfinite(got.float()).all(), f"call {call}: output not written"
        # the same kernels with the same split: the same bits as the ordinary entry point
        assert torch.equal(got, want), f"call {call}: differs from the ordinary entry point"
        # and right by itself, against a plain float64 attention
        for b, n in enumerate(lens):
            ref = attention_reference(q[b].cpu().view(nh, HD), pc.k[b], pc.v[b], n - 1, window or None, scale)
            assert torch.allclose(got[b].cpu().double().view(nh, HD), ref, rtol=2e-2, atol=2e-2), \
                f"call {call}, sequence {b}"

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
