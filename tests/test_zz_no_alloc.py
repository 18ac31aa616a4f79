"""The allocation-free decode attention entry point, called the way a C program
would call it: through its exported symbol, with raw device pointers.

Some users of this library cannot allocate device memory when they need attention
(every buffer was sized at start-up, or the caller is plain C with no allocator
to borrow from), so `aie_paged_attention_decode_noalloc` keeps its scratch in a
fixed 16 MiB array inside the library.  Here its output is compared with the
regular entry point's (which takes scratch from the caller) on two calls in a
row with different inputs — the second call finds the first call's leftovers in
the shared array and must not be disturbed by them — and a call that would need
more than the array holds must be refused without launching anything.
This file is collected last, so a run that stops at the first failure has
already run every other test.
"""
import ctypes
import math
from ctypes import c_float, c_int, c_void_p

import pytest
import torch

from test_kernels_gpu import DEV, attention_reference, err_word, ops, paged_setup

pytestmark = pytest.mark.gpu

TOL = 2e-2      # the bfloat16 attention tolerance of tests/test_kernels_gpu.py


def noalloc_lib():
    from ai_engine_b200.csrc.build import cuda_library

    lib = ctypes.CDLL(cuda_library("attention_decode_noalloc.cu"))
    fn = lib.aie_paged_attention_decode_noalloc
    fn.restype = c_int
    return fn


def call_noalloc(fn, s, H, K, d, window, splits, out, e):
    P = s["k_pages"].shape[2]
    dec = torch.arange(len(s["lens"]), device=DEV, dtype=torch.int32)
    p = lambda t: c_void_p(t.data_ptr())
    return fn(p(s["q"]), p(s["k_pages"]), p(s["v_pages"]), p(out), p(dec), c_int(dec.shape[0]),
              p(s["positions"]), p(s["token_req"]), p(s["bt"]), c_int(s["bt"].shape[1]),
              c_int(s["k_pages"].shape[0]), c_int(P), c_int(H), c_int(K), c_int(d), c_int(window),
              c_float(1.0 / math.sqrt(d)), c_int(splits), p(e),
              c_void_p(torch.cuda.current_stream().cuda_stream))


def test_noalloc_entry_point_matches_the_regular_one_twice_in_a_row():
    fn = noalloc_lib()
    calls = [  # H, K, d, P, lens, window, splits, seed — the second differs in every size
        (32, 8, 128, 16, [1024, 3, 517, 90], 0, 4, 1),
        (6, 2, 64, 8, [33, 257, 700], 20, 6, 2),
    ]
    for H, K, d, P, lens, window, splits, seed in calls:
        s = paged_setup(torch.bfloat16, H, K, d, P, lens, [1] * len(lens), seed=seed)
        e = err_word()
        got = torch.full_like(s["q"], float("nan"))
        before = torch.cuda.memory_allocated()
        rc = call_noalloc(fn, s, H, K, d, window, splits, got, e)
        assert rc == 0
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        want = torch.full_like(s["q"], float("nan"))
        dec = torch.arange(len(lens), device=DEV, dtype=torch.int32)
        ops().paged_attention_decode(s["q"], s["k_pages"], s["v_pages"], dec, s["positions"], s["token_req"],
                                     s["bt"], 1.0 / math.sqrt(d), window, splits, e, want)
        assert int(e.item()) == 0 and not torch.isnan(got).any()
        assert (got.float() - want.float()).abs().max() <= TOL
        ref = attention_reference(s, H, K, d, 1.0 / math.sqrt(d), window)
        assert (got.double() - ref).abs().max() <= TOL


def test_noalloc_entry_point_refuses_what_its_scratch_cannot_hold():
    fn = noalloc_lib()
    H, K, d = 32, 8, 128
    lens = [40] * 40
    s = paged_setup(torch.bfloat16, H, K, d, 16, lens, [1] * len(lens), seed=3)
    out = torch.full_like(s["q"], 7.0)
    e = err_word()
    # 40 requests x 32 heads x 32 parts x 129 floats = 5.3 M floats > 4 Mi
    assert call_noalloc(fn, s, H, K, d, 0, 32, out, e) == -3
    torch.cuda.synchronize()
    assert bool((out == 7.0).all())                       # nothing was launched
    assert call_noalloc(fn, s, H, K, d, 0, 1, out, e) == 0     # one part needs no scratch
    torch.cuda.synchronize()
    ref = attention_reference(s, H, K, d, 1.0 / math.sqrt(d), 0)
    assert (out.double() - ref).abs().max() <= TOL
